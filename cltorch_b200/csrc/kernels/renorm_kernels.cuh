// Row-wise renorm in one pass for rows that fit in the registers of a warp or a CTA (up to 16384 elements): the row is
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

// sum^(1/p), rounded to fp32 from a double-precision root (pow in double costs a few hundred instructions,
// which short rows would notice: p = 1, 2, 3 take the exact, square and cube root instead).
template <int PMODE>
__device__ __forceinline__ float thb_rnf_root(float sum, float p) {
  if (PMODE == 1) return sum;
  if (PMODE == 2) return (float)sqrt((double)sum);
  if (PMODE == 3) return (float)cbrt((double)sum);
  return thb_pow(sum, 1.0f / p);
}

// Whether a row whose sum of |x|^p is `sum` is rescaled (not for a NaN norm), and by what.
template <int PMODE>
__device__ __forceinline__ bool thb_rnf_factor(double sum, float p, float maxnorm, float* f) {
  const float norm = thb_rnf_root<PMODE>((float)sum, p);
  if (!(norm > maxnorm)) return false;
  *f = (float)((double)maxnorm / ((double)norm + 1e-7));
  return true;
}

// A group of L lanes (8, 16 or 32) takes R rows of at most 4 * L * U elements at a time, so a lane has R * U = 8
// (16 when U = 16) vectors in flight and a warp works on R * 32 / L rows. The factor of row r of a group is
// worked out by the group's lane r (one pass through the root for all rows of the warp) and handed round.
template <int L, int U, int R, int PMODE>
__global__ void __launch_bounds__(THB_RNF_THREADS, 2)
thb_renorm_rows_warp(float* data, thb_i64 rows, thb_u32 size, float p, float maxnorm) {
  static_assert(R <= L, "lane r of a group serves row r");
  constexpr int kGroups = 32 / L;
  const int lane = threadIdx.x & 31, sub = lane % L, group = lane / L;
  const thb_u32 nvec = size >> 2;
  const thb_i64 per_warp = (thb_i64)R * kGroups;
  const thb_i64 warps = (thb_i64)gridDim.x * (THB_RNF_THREADS / 32);
  for (thb_i64 row0 = ((thb_i64)blockIdx.x * (THB_RNF_THREADS / 32) + (threadIdx.x >> 5)) * per_warp; row0 < rows;
       row0 += warps * per_warp) {
    float4 v[R][U];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const thb_i64 row = row0 + r * kGroups + group;
      const float4* r4 = reinterpret_cast<const float4*>(data + row * (thb_i64)size);
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const thb_u32 i = j * L + sub;
        v[r][j] = (row < rows && i < nvec) ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    double acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      acc[r] = 0.0;
#pragma unroll
      for (int j = 0; j < U; ++j)
        if (j * L + sub < nvec) acc[r] += thb_rnf_terms<PMODE>(v[r][j], p);
    }
#pragma unroll
    for (int off = L / 2; off > 0; off >>= 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
    }
    double mine = 0.0;
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (sub == r) mine = acc[r];
    float f_mine = 1.f;
    const int scale_mine = thb_rnf_factor<PMODE>(mine, p, maxnorm, &f_mine) ? 1 : 0;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float f = __shfl_sync(0xffffffffu, f_mine, group * L + r);
      const int scale = __shfl_sync(0xffffffffu, scale_mine, group * L + r);
      const thb_i64 row = row0 + r * kGroups + group;
      if (row < rows && scale) {
        float4* r4 = reinterpret_cast<float4*>(data + row * (thb_i64)size);
#pragma unroll
        for (int j = 0; j < U; ++j) {
          const thb_u32 i = j * L + sub;
          if (i < nvec) r4[i] = make_float4(v[r][j].x * f, v[r][j].y * f, v[r][j].z * f, v[r][j].w * f);
        }
      }
    }
  }
}

// One CTA of THREADS threads per row of at most 64 * THREADS elements: 16 vectors in flight per thread, and as many
// CTAs per SM as the registers allow (2 of 256 threads, 4 of 128, 8 of 64), so 128 KB of loads per SM either way.
#define THB_RNF_BLOCK_U 16
template <int THREADS, int PMODE>
__global__ void __launch_bounds__(THREADS, 512 / THREADS)
thb_renorm_rows_block(float* data, thb_i64 rows, thb_u32 size, float p, float maxnorm) {
  constexpr int U = THB_RNF_BLOCK_U;
  __shared__ double smem[32];
  __shared__ float s_factor;
  __shared__ int s_scale;
  const thb_u32 nvec = size >> 2;
  for (thb_i64 row = blockIdx.x; row < rows; row += gridDim.x) {
    float4* r4 = reinterpret_cast<float4*>(data + row * (thb_i64)size);
    float4 v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const thb_u32 i = j * THREADS + threadIdx.x;
      v[j] = i < nvec ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    double acc[2] = {0.0, 0.0};
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (j * THREADS + threadIdx.x < nvec) acc[j & 1] += thb_rnf_terms<PMODE>(v[j], p);
    const double total = thb_block_fold<RedAdd>(acc[0] + acc[1], 0.0, smem);
    if (threadIdx.x == 0) {
      float f0 = 1.f;
      s_scale = thb_rnf_factor<PMODE>(total, p, maxnorm, &f0) ? 1 : 0;
      s_factor = f0;
    }
    __syncthreads();
    const float f = s_factor;
    if (s_scale) {
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const thb_u32 i = j * THREADS + threadIdx.x;
        if (i < nvec) r4[i] = make_float4(v[j].x * f, v[j].y * f, v[j].z * f, v[j].w * f);
      }
    }
    __syncthreads();  // s_factor, s_scale and smem are reused by the next row
  }
}
