// Level-1/2 BLAS kernels behind dot and addmv: all bound by HBM (each matrix or
// vector element is read once), accumulated in double and rounded to fp32 once.
// They stand in for clblasSdot and clblasSgemv as called from the reference's
// src/lib/THClBlas.cpp:149-262 (column-major conventions).
#pragma once
#include "reduce_kernels.cuh"

// partial[b] = sum over this block's share of a[i] * b[i]; folded by thb_reduce_all_pass2<RedAdd>.
__global__ void __launch_bounds__(THB_RA_THREADS, THB_RA_BLOCKS_PER_SM)
thb_dot_pass1(const float* a, const float* b, thb_i64 n, int vec_ok, double* partials) {
  __shared__ double smem[32];
  double acc[4] = {0.0, 0.0, 0.0, 0.0};
  if (vec_ok) {
    const thb_i64 nvec = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    const thb_i64 step = (thb_i64)gridDim.x * (THB_RA_THREADS * 4);
    for (thb_i64 base = (thb_i64)blockIdx.x * (THB_RA_THREADS * 4) + threadIdx.x; base < nvec; base += step) {
      float4 x[4], y[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        thb_i64 i = base + u * THB_RA_THREADS;
        if (i < nvec) { x[u] = a4[i]; y[u] = b4[i]; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        thb_i64 i = base + u * THB_RA_THREADS;
        if (i < nvec) {
          acc[0] = fma((double)x[u].x, (double)y[u].x, acc[0]);
          acc[1] = fma((double)x[u].y, (double)y[u].y, acc[1]);
          acc[2] = fma((double)x[u].z, (double)y[u].z, acc[2]);
          acc[3] = fma((double)x[u].w, (double)y[u].w, acc[3]);
        }
      }
    }
    if (blockIdx.x == 0 && threadIdx.x < (int)(n & 3)) {
      thb_i64 i = (nvec << 2) + threadIdx.x;
      acc[0] = fma((double)a[i], (double)b[i], acc[0]);
    }
  } else {
    const thb_i64 step = (thb_i64)gridDim.x * THB_RA_THREADS;
    for (thb_i64 i = (thb_i64)blockIdx.x * THB_RA_THREADS + threadIdx.x; i < n; i += step) acc[0] = fma((double)a[i], (double)b[i], acc[0]);
  }
  double r = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  r = thb_block_fold<RedAdd>(r, 0.0, smem);
  if (threadIdx.x == 0) partials[blockIdx.x] = r;
}

// y[j] = alpha * sum_i A[i + j*lda] * x[i*incx] + beta * y[j*incy], j < n: every
// output is a dot product with one contiguous column of A (length m). One warp
// per output (WARP) or one block per output.
template <bool WARP>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_gemv_t(const float* A, thb_i64 lda, const float* x, thb_i64 incx, float* y, thb_i64 incy, thb_u32 m, thb_u32 n,
           float alpha, float beta) {
  __shared__ double smem[32];
  const int lane = threadIdx.x & 31;
  const int t = WARP ? lane : (int)threadIdx.x;
  const int nt = WARP ? 32 : THB_RD_THREADS;
  const thb_u32 per_block = WARP ? THB_RD_THREADS / 32 : 1;
  for (thb_u64 j0 = (thb_u64)blockIdx.x * per_block; j0 < n; j0 += (thb_u64)gridDim.x * per_block) {
    const thb_u64 j = WARP ? j0 + (threadIdx.x >> 5) : j0;
    double acc = 0.0;
    if (j < n) {
      const float* col = A + j * lda;
      if (incx == 1 && ((((thb_u64)col) | ((thb_u64)x)) & 15) == 0 && (m & 3) == 0) {
        const float4* c4 = reinterpret_cast<const float4*>(col);
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (thb_u32 i = t; i < (m >> 2); i += nt) {
          float4 a = c4[i], b = x4[i];
          acc = fma((double)a.x, (double)b.x, acc);
          acc = fma((double)a.y, (double)b.y, acc);
          acc = fma((double)a.z, (double)b.z, acc);
          acc = fma((double)a.w, (double)b.w, acc);
        }
      } else {
        for (thb_u32 i = t; i < m; i += nt) acc = fma((double)col[i], (double)x[(thb_i64)i * incx], acc);
      }
    }
    if (WARP) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(THB_FULL_MASK, acc, off);
      if (lane == 0 && j < n) {
        float r = alpha * (float)acc;
        if (beta != 0.f) r += beta * y[j * incy];
        y[j * incy] = r;
      }
    } else {
      acc = thb_block_fold<RedAdd>(acc, 0.0, smem);
      if (threadIdx.x == 0) {
        float r = alpha * (float)acc;
        if (beta != 0.f) r += beta * y[j * incy];
        y[j * incy] = r;
      }
      __syncthreads();
    }
  }
}

// y[i] = alpha * sum_j A[i + j*lda] * x[j*incx] + beta * y[i*incy], i < m: A is read
// along its unit-stride dimension by adjacent threads; the sum over j is cut into
// gridDim.y chunks (partial[chunk * m + i]) when m alone cannot fill the GPU.
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_gemv_n(const float* A, thb_i64 lda, const float* x, thb_i64 incx, float* y, thb_i64 incy, thb_u32 m, thb_u32 n,
           float alpha, float beta, thb_u32 chunk_len, thb_u32 nchunks, double* partial) {
  const thb_u32 chunk = blockIdx.y;
  const thb_u32 j0 = chunk * chunk_len, j1 = min(n, j0 + chunk_len);
  for (thb_u64 i = (thb_u64)blockIdx.x * THB_RD_THREADS + threadIdx.x; i < m; i += (thb_u64)gridDim.x * THB_RD_THREADS) {
    const float* p = A + i;
    double acc = 0.0;
    thb_u32 j = j0;
    for (; j + 8 <= j1; j += 8) {
      float a[8], b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) { a[u] = p[(thb_i64)(j + u) * lda]; b[u] = x[(thb_i64)(j + u) * incx]; }
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = fma((double)a[u], (double)b[u], acc);
    }
    for (; j < j1; ++j) acc = fma((double)p[(thb_i64)j * lda], (double)x[(thb_i64)j * incx], acc);
    if (nchunks == 1) {
      float r = alpha * (float)acc;
      if (beta != 0.f) r += beta * y[i * incy];
      y[i * incy] = r;
    } else {
      partial[(thb_u64)chunk * m + i] = acc;
    }
  }
}

__global__ void __launch_bounds__(THB_RD_THREADS)
thb_gemv_n_fold(const double* partial, float* y, thb_i64 incy, thb_u32 m, thb_u32 nchunks, float alpha, float beta) {
  for (thb_u64 i = (thb_u64)blockIdx.x * THB_RD_THREADS + threadIdx.x; i < m; i += (thb_u64)gridDim.x * THB_RD_THREADS) {
    double acc = 0.0;
    for (thb_u32 c = 0; c < nchunks; ++c) acc += partial[(thb_u64)c * m + i];
    float r = alpha * (float)acc;
    if (beta != 0.f) r += beta * y[i * incy];
    y[i * incy] = r;
  }
}
