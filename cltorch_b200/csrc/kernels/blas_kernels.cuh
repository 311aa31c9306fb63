// Level-1/2 BLAS kernels behind dot, addmv and addr: all bound by HBM (each matrix or
// vector element is read once). Products are rounded to fp32 (as clBLAS does), their sum is
// kept in double and rounded to fp32 once: one fp32 -> fp64 conversion per element. The
// conversions run on the quarter-rate XU pipe, and with exact products in double (two
// conversions per element) that pipe, not HBM, set the pace (61 % busy at 0.78 of the HBM rate).
// They stand in for clblasSdot and clblasSgemv as called from the reference's
// src/lib/THClBlas.cpp:149-262 (column-major conventions).
#pragma once
#include "reduce_strip_kernels.cuh"

// partial[b] = sum over this block's share of a[i] * b[i]; the block that finishes last folds the
// partials (F.ticket), or thb_reduce_all_pass2<RedAdd> does when there is no ticket.
__global__ void __launch_bounds__(THB_RA_THREADS, THB_RA_BLOCKS_PER_SM)
thb_dot_pass1(const float* a, const float* b, thb_i64 n, int vec_ok, double* partials, ThbFinish F) {
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
          acc[0] += (double)(x[u].x * y[u].x);
          acc[1] += (double)(x[u].y * y[u].y);
          acc[2] += (double)(x[u].z * y[u].z);
          acc[3] += (double)(x[u].w * y[u].w);
        }
      }
    }
    if (blockIdx.x == 0 && threadIdx.x < (int)(n & 3)) {
      thb_i64 i = (nvec << 2) + threadIdx.x;
      acc[0] += (double)(a[i] * b[i]);
    }
  } else {
    const thb_i64 step = (thb_i64)gridDim.x * THB_RA_THREADS;
    for (thb_i64 i = (thb_i64)blockIdx.x * THB_RA_THREADS + threadIdx.x; i < n; i += step) acc[0] += (double)(a[i] * b[i]);
  }
  double r = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  r = thb_block_fold<RedAdd>(r, 0.0, smem);
  if (threadIdx.x == 0) partials[blockIdx.x] = r;
  if (F.ticket) thb_finish_last_block<RedAdd>(F, partials, 0.f, smem);
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
        // 4 vectors of the column and of x in flight per thread, one accumulator per vector lane;
        // the matrix goes past L1 so that x, which every column needs again, stays there
        const float4* c4 = reinterpret_cast<const float4*>(col);
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const thb_u32 nvec = m >> 2;
        double a4[4] = {0.0, 0.0, 0.0, 0.0};
        for (thb_u32 i = t; i < nvec; i += nt * 4) {
          float4 a[4], b[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i + u * nt < nvec) { a[u] = __ldcg(c4 + i + u * nt); b[u] = x4[i + u * nt]; }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i + u * nt < nvec) {
              a4[0] += (double)(a[u].x * b[u].x);
              a4[1] += (double)(a[u].y * b[u].y);
              a4[2] += (double)(a[u].z * b[u].z);
              a4[3] += (double)(a[u].w * b[u].w);
            }
        }
        acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
      } else {
        for (thb_u32 i = t; i < m; i += nt) acc += (double)(col[i] * x[(thb_i64)i * incx]);
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
      for (int u = 0; u < 8; ++u) acc += (double)(a[u] * b[u]);
    }
    for (; j < j1; ++j) acc += (double)(p[(thb_i64)j * lda] * x[(thb_i64)j * incx]);
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

// y = alpha * A x + beta * y through the TMA strip pipeline: a strip is 128 consecutive outputs
// i (the unit-stride direction of A), the rows of the strip are the columns j of A, and every
// row is weighted by x[j]. Two threads per output (even / odd j), four accumulators each; the
// partials are folded by thb_gemv_n_fold.
struct ThbGemvConsumer {
  static constexpr bool kRowWeights = true;  // x[j], staged in shared memory by the producer warp
  struct Params {
    const float* x;
    thb_i64 incx;
    double* partial;   // [npartials][m]
  };
  double acc[4];
  static __device__ __forceinline__ float weight(const Params& p, thb_u32 j) { return p.x[(thb_i64)j * p.incx]; }
  __device__ __forceinline__ void begin(const Params&, const ThbStripGeom&, int, thb_i64, bool, int) {
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] = 0.0;
  }
  __device__ __forceinline__ void row(float v, thb_u32, int slot, float xj) { acc[slot] += (double)(v * xj); }
  __device__ __forceinline__ void end(const Params& p, const ThbStripGeom& g, int, thb_i64 col, int part) {
    p.partial[(thb_u64)part * g.nslices + col] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  }
};

// Rank-1 update of a matrix with unit-stride rows, c in vectors of 4:
//   ALPHA_ON_ROW:  A[r * lda + c] += (alpha * vr[r * incr]) * vc[c]
//   otherwise:     A[r * lda + c] += (alpha * vc[c]) * vr[r * incr]
// (the operator "*out += val1 * *in1 * *in2" rounds alpha * in1 first: which of the two vectors is
// in1 depends on whether the result or its transpose has the unit-stride rows).
// clblasSger as called from THClBlas_ger (reference src/lib/THClBlas.cpp:264-347).
template <bool ALPHA_ON_ROW>
__global__ void __launch_bounds__(256)
thb_ger_rows(float* A, thb_i64 lda, thb_u32 rows, thb_u32 cvec, const float* vr, thb_i64 incr, const float* vc, float alpha) {
  const thb_u64 nvec = (thb_u64)rows * cvec;
  const float4* vc4 = reinterpret_cast<const float4*>(vc);
  for (thb_u64 base = (thb_u64)blockIdx.x * 1024 + threadIdx.x; base < nvec; base += (thb_u64)gridDim.x * 1024) {
    float4 a[4], c[4];
    float s[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const thb_u64 i = base + u * 256;
      if (i < nvec) {
        const thb_u32 r = (thb_u32)(i / cvec), q = (thb_u32)(i - (thb_u64)r * cvec);
        a[u] = *reinterpret_cast<const float4*>(A + (thb_i64)r * lda + 4 * (thb_i64)q);
        c[u] = vc4[q];
        s[u] = vr[(thb_i64)r * incr];
        if (ALPHA_ON_ROW) s[u] = alpha * s[u];
        else { c[u].x = alpha * c[u].x; c[u].y = alpha * c[u].y; c[u].z = alpha * c[u].z; c[u].w = alpha * c[u].w; }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const thb_u64 i = base + u * 256;
      if (i < nvec) {
        const thb_u32 r = (thb_u32)(i / cvec), q = (thb_u32)(i - (thb_u64)r * cvec);
        a[u].x += s[u] * c[u].x; a[u].y += s[u] * c[u].y; a[u].z += s[u] * c[u].z; a[u].w += s[u] * c[u].w;
        *reinterpret_cast<float4*>(A + (thb_i64)r * lda + 4 * (thb_i64)q) = a[u];
      }
    }
  }
}
