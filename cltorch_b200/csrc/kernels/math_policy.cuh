// Accuracy policy for the transcendental functions used by pointwise operators.
//
// FREESTANDING like apply_kernels.cuh: compiled by nvcc and by NVRTC.
//
// Pointwise results must agree with a correctly rounded fp32 evaluation to
// within 2 ulp. CUDA's single-precision tanf, sinhf, atan2f and powf are
// documented at 3-4 ulp, so those are evaluated in double and rounded once;
// the others use the fp32 library routine (<= 2 ulp documented, IEEE sqrt and
// division since the build uses neither fast-math nor fused multiply-add).
#pragma once

__device__ __forceinline__ float thb_log(float x) { return logf(x); }
__device__ __forceinline__ float thb_log1p(float x) { return log1pf(x); }
__device__ __forceinline__ float thb_exp(float x) { return expf(x); }
__device__ __forceinline__ float thb_cos(float x) { return cosf(x); }
__device__ __forceinline__ float thb_sin(float x) { return sinf(x); }
__device__ __forceinline__ float thb_acos(float x) { return acosf(x); }
__device__ __forceinline__ float thb_asin(float x) { return asinf(x); }
__device__ __forceinline__ float thb_atan(float x) { return atanf(x); }
__device__ __forceinline__ float thb_cosh(float x) { return coshf(x); }
__device__ __forceinline__ float thb_tanh(float x) { return tanhf(x); }
__device__ __forceinline__ float thb_tan(float x) { return (float)tan((double)x); }
__device__ __forceinline__ float thb_sinh(float x) { return (float)sinh((double)x); }
__device__ __forceinline__ float thb_atan2(float y, float x) { return (float)atan2((double)y, (double)x); }
__device__ __forceinline__ float thb_pow(float x, float y) { return (float)pow((double)x, (double)y); }
// OpenCL pown(x, n): integer exponent, defined for negative bases
// (reference src/lib/THClTensorMath2.cpp:22-44 selects it when the exponent is integer-valued).
__device__ __forceinline__ float thb_pown(float x, float n) { return (float)pow((double)x, (double)(int)n); }
