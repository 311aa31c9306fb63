// Accuracy policy for the transcendental functions used by pointwise operators.
//
// FREESTANDING like apply_kernels.cuh: compiled by nvcc and by NVRTC.
//
// Pointwise results must agree with a correctly rounded fp32 evaluation to
// within 2 ulp. CUDA's single-precision tanf, sinhf, atan2f and powf are
// documented at 3-4 ulp, so those are evaluated in double and rounded once; so
// is exp, because it feeds composites (sigmoid = 1 / (1 + exp(-x)) measured 4 ulp
// with expf). The others use the fp32 library routine (<= 2 ulp documented, IEEE
// sqrt and division since the build uses neither fast-math nor fused multiply-add).
#pragma once

__device__ __forceinline__ float thb_log(float x) { return logf(x); }
__device__ __forceinline__ float thb_log1p(float x) { return log1pf(x); }
__device__ __forceinline__ float thb_exp(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float thb_cos(float x) { return cosf(x); }
__device__ __forceinline__ float thb_sin(float x) { return sinf(x); }
__device__ __forceinline__ float thb_acos(float x) { return acosf(x); }
__device__ __forceinline__ float thb_asin(float x) { return asinf(x); }
__device__ __forceinline__ float thb_atan(float x) { return atanf(x); }
__device__ __forceinline__ float thb_cosh(float x) { return coshf(x); }
// Reciprocal seed in double, good to about 20 bits (one Newton step then gives 40): the
// special-function unit's approximation, which spares the two fp64 <-> fp32 conversions
// that a float reciprocal would cost.
__device__ __forceinline__ double thb_rcp_seed(double d) {
  double y;
  asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(y) : "d"(d));
  return y;
}
// tanh to within 1 ulp, so that products such as tanh(x)*x stay within 2 ulp of a
// correctly rounded evaluation (tanhf alone is documented at 2 ulp and measured
// 3 ulp in that product). |x| <= 1 uses a Pade approximant in double; beyond that,
// em = expm1(2|x|) in double from a degree-9 polynomial
// after the usual ln2 range reduction (relative error < 1e-12), then
// em / (em + 2) with an approximate reciprocal refined by one Newton step in double:
// about 25 fp64 instructions, a fraction of the library tanh(double).
__device__ __forceinline__ float thb_tanh(float xf) {
  const float ax = fabsf(xf);
  if (!(ax <= 20.0f)) return (ax != ax) ? xf : copysignf(1.0f, xf);  // NaN, or saturated
  if (ax < 2.44140625e-4f) return fmaf(xf * xf * xf, -0.333333343f, xf);  // |x| < 2^-12: x - x^3/3
  if (ax <= 1.0f) {
    // |x| <= 1: the [7/6] Pade approximant x*(135135 + 17325 x^2 + 378 x^4 + x^6) /
    // (135135 + 62370 x^2 + 3150 x^4 + 28 x^6), relative error < 3e-12 on this range,
    // about 11 fp64 instructions
    const double x = (double)xf, q = x * x;
    const double num = x * fma(fma(fma(q, 1.0, 378.0), q, 17325.0), q, 135135.0);
    const double den = fma(fma(fma(q, 28.0, 3150.0), q, 62370.0), q, 135135.0);
    double y = thb_rcp_seed(den);
    y = y * fma(-den, y, 2.0);
    return (float)(num * y);
  }
  const double x2 = 2.0 * (double)ax;
  const double n = rint(x2 * 1.4426950408889634);
  double r = fma(n, -6.93147180369123816490e-01, x2);
  r = fma(n, -1.90821492927058770002e-10, r);
  double p = 2.7557319223985893e-07;            // 1/10!
  p = fma(p, r, 2.7557319223985888e-06);        // 1/9!
  p = fma(p, r, 2.4801587301587302e-05);        // 1/8!
  p = fma(p, r, 1.9841269841269841e-04);        // 1/7!
  p = fma(p, r, 1.3888888888888889e-03);        // 1/6!
  p = fma(p, r, 8.3333333333333332e-03);        // 1/5!
  p = fma(p, r, 4.1666666666666664e-02);        // 1/4!
  p = fma(p, r, 1.6666666666666666e-01);        // 1/3!
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  const double pm = p * r;                      // expm1(r)
  const double s = __longlong_as_double(((long long)n + 1023ll) << 52);  // 2^n, 0 <= n <= 58
  const double em = fma(s, pm, s - 1.0);        // expm1(2|x|)
  const double d = em + 2.0;
  double y = thb_rcp_seed(d);
  y = y * fma(-d, y, 2.0);
  return copysignf((float)(em * y), xf);
}
__device__ __forceinline__ float thb_tan(float x) { return (float)tan((double)x); }
__device__ __forceinline__ float thb_sinh(float x) { return (float)sinh((double)x); }
__device__ __forceinline__ float thb_atan2(float y, float x) { return (float)atan2((double)y, (double)x); }
__device__ __forceinline__ float thb_pow(float x, float y) { return (float)pow((double)x, (double)y); }
// OpenCL pown(x, n): integer exponent, defined for negative bases
// (reference src/lib/THClTensorMath2.cpp:22-44 selects it when the exponent is integer-valued).
__device__ __forceinline__ float thb_pown(float x, float n) { return (float)pow((double)x, (double)(int)n); }
