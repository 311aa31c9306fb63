// Row-wise renorm in one pass for rows that fit in the registers of a warp or a CTA: the row is
// loaded once, its p-norm is folded in double, and the registers are written back scaled only
// when the norm exceeds the limit. HBM traffic: 4 bytes per element read, 4 more written for
// the rows that are rescaled (the two-kernel form, a row reduction followed by thb_renorm_scale,
// reads those rows a second time: 4 + 8).
//
// Same job as THClTensor_kernel_renorm (reference src/lib/THClTensorMath2.cl:110-143): row r of
// data ([rows][size], contiguous) is multiplied by maxnorm / (norm + 1e-7) when
// norm = (sum |x|^p)^(1/p) exceeds maxnorm, and left untouched otherwise.
//
// Rows are 16-byte aligned and a multiple of 4 long here; other layouts take the two-kernel form.
#pragma once
#include "math_policy.cuh"
#include "reduce_kernels.cuh"

#define THB_RNF_THREADS 256

// PMODE 1, 2, 3: |x|, x^2, |x|^3 without a comparison of p per element; 0: the general power.
template <int PMODE>
__device__ __forceinline__ float thb_rnf_term(float x, float p) {
  if (PMODE == 1) return fabsf(x);
  if (PMODE == 2) return x * x;
  if (PMODE == 3) return fabsf(x) * (x * x);
  return thb_abs_pow_general(x, p);
}

template <int PMODE>
__device__ __forceinline__ double thb_rnf_terms(const float4& v, float p) {
  return ((double)thb_rnf_term<PMODE>(v.x, p) + (double)thb_rnf_term<PMODE>(v.y, p)) +
         ((double)thb_rnf_term<PMODE>(v.z, p) + (double)thb_rnf_term<PMODE>(v.w, p));
}

// Whether a row whose sum of |x|^p is `sum` is rescaled (not for a NaN norm), and by what.
__device__ __forceinline__ bool thb_rnf_factor(double sum, float p, float maxnorm, float* f) {
  const float norm = thb_pow((float)sum, 1.0f / p);
  if (!(norm > maxnorm)) return false;
  *f = (float)((double)maxnorm / ((double)norm + 1e-7));
  return true;
}

// One warp per row of at most 128 * U elements.
template <int U, int PMODE>
__global__ void __launch_bounds__(THB_RNF_THREADS)
thb_renorm_rows_warp(float* data, thb_i64 rows, thb_u32 size, float p, float maxnorm) {
  const int lane = threadIdx.x & 31;
  const thb_u32 nvec = size >> 2;
  const thb_i64 warps = (thb_i64)gridDim.x * (THB_RNF_THREADS / 32);
  for (thb_i64 row = (thb_i64)blockIdx.x * (THB_RNF_THREADS / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    float4* r4 = reinterpret_cast<float4*>(data + row * (thb_i64)size);
    float4 v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const thb_u32 i = j * 32 + lane;
      v[j] = i < nvec ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    double acc = 0.0;
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (j * 32 + lane < nvec) acc += thb_rnf_terms<PMODE>(v[j], p);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    float f = 1.f;
    if (thb_rnf_factor(acc, p, maxnorm, &f)) {
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const thb_u32 i = j * 32 + lane;
        if (i < nvec) r4[i] = make_float4(v[j].x * f, v[j].y * f, v[j].z * f, v[j].w * f);
      }
    }
  }
}

// One CTA per row of at most 1024 * U elements.
template <int U, int PMODE>
__global__ void __launch_bounds__(THB_RNF_THREADS, 2)
thb_renorm_rows_block(float* data, thb_i64 rows, thb_u32 size, float p, float maxnorm) {
  __shared__ double smem[32];
  __shared__ float s_factor;
  __shared__ int s_scale;
  const thb_u32 nvec = size >> 2;
  for (thb_i64 row = blockIdx.x; row < rows; row += gridDim.x) {
    float4* r4 = reinterpret_cast<float4*>(data + row * (thb_i64)size);
    float4 v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const thb_u32 i = j * THB_RNF_THREADS + threadIdx.x;
      v[j] = i < nvec ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    double acc[2] = {0.0, 0.0};
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (j * THB_RNF_THREADS + threadIdx.x < nvec) acc[j & 1] += thb_rnf_terms<PMODE>(v[j], p);
    const double total = thb_block_fold<RedAdd>(acc[0] + acc[1], 0.0, smem);
    if (threadIdx.x == 0) {
      float f0 = 1.f;
      s_scale = thb_rnf_factor(total, p, maxnorm, &f0) ? 1 : 0;
      s_factor = f0;
    }
    __syncthreads();
    const float f = s_factor;
    if (s_scale) {
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const thb_u32 i = j * THB_RNF_THREADS + threadIdx.x;
        if (i < nvec) r4[i] = make_float4(v[j].x * f, v[j].y * f, v[j].z * f, v[j].w * f);
      }
    }
    __syncthreads();  // s_factor, s_scale and smem are reused by the next row
  }
}
