// Inclusive scans (cumsum, cumprod) along one dimension, the row-wise renorm scaling
// and the p-distance of two vectors, for sm_100a.
//
// They replace THClTensor_kernel_scanOuterDim / scanInnermostDim
// (reference src/lib/THClTensorMathScan.cl:27-139), THClTensor_kernel_renorm
// (src/lib/THClTensorMath2.cl:110-143) and the thrust::inner_product of
// THClTensor_dist (src/lib/THClTensorMath2.cpp:448-475).
//
// A scanned tensor is contiguous and viewed as [outer][n][inner]; the scan runs
// along n. All kernels are bound by HBM: 8 bytes per element when one pass is
// enough, 12 when the scanned dimension has to be cut into chunks to fill the
// GPU (chunk totals, a scan of the totals, then the scan proper with a carry-in).
// Running values are kept in double and rounded to fp32 at each store.
#pragma once
#include "reduce_kernels.cuh"

#define THB_SC_THREADS 256
#define THB_SC_ROW_UNROLL 4

struct ScanAdd {
  static __device__ __forceinline__ double identity() { return 0.0; }
  static __device__ __forceinline__ double apply(double a, double b) { return a + b; }
};
struct ScanMul {
  static __device__ __forceinline__ double identity() { return 1.0; }
  static __device__ __forceinline__ double apply(double a, double b) { return a * b; }
};

// carry / totals layout: [outer][nchunks][inner] doubles

// inner > 1: one thread per VEC adjacent inner positions and chunk (blockIdx.y) walks the
// rows of its chunk; adjacent threads read adjacent addresses. TOTALS: only the chunk total
// is produced (phase 1 of a chunked scan), nothing is stored to dst.
#define THB_SC_COLS_BLOCKS 4  // resident blocks per SM of thb_scan_cols (<= 64 registers)
template <class Op, int VEC, bool TOTALS>
__global__ void __launch_bounds__(THB_SC_THREADS, THB_SC_COLS_BLOCKS)
thb_scan_cols(float* dst, const float* src, thb_i64 outer, thb_u32 n, thb_i64 inner, thb_u32 chunk_len,
              thb_u32 nchunks, double* carry) {
  const thb_u32 chunk = blockIdx.y;
  const thb_u32 r0 = chunk * chunk_len;
  const thb_u32 r1 = min(n, r0 + chunk_len);
  const thb_i64 per_outer = inner / VEC;
  const thb_i64 total = outer * per_outer;
  for (thb_i64 q = (thb_i64)blockIdx.x * THB_SC_THREADS + threadIdx.x; q < total;
       q += (thb_i64)gridDim.x * THB_SC_THREADS) {
    const thb_i64 o = q / per_outer, i = (q - o * per_outer) * VEC;
    const thb_i64 base = o * (thb_i64)n * inner + i;
    const thb_i64 cbase = (o * nchunks + chunk) * inner + i;
    double acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = (!TOTALS && nchunks > 1) ? carry[cbase + j] : Op::identity();
    thb_u32 r = r0;
    for (; r + 8 <= r1; r += 8) {
      float v[8][VEC];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float* p = src + base + (thb_i64)(r + u) * inner;
        if (VEC == 4) {
          const float4 t = *reinterpret_cast<const float4*>(p);
          v[u][0] = t.x; v[u][1 % VEC] = t.y; v[u][2 % VEC] = t.z; v[u][3 % VEC] = t.w;
        } else {
          v[u][0] = *p;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float o4[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          acc[j] = Op::apply(acc[j], (double)v[u][j]);
          o4[j] = (float)acc[j];
        }
        if (!TOTALS) {
          float* d = dst + base + (thb_i64)(r + u) * inner;
          if (VEC == 4) *reinterpret_cast<float4*>(d) = make_float4(o4[0], o4[1 % VEC], o4[2 % VEC], o4[3 % VEC]);
          else *d = o4[0];
        }
      }
    }
    for (; r < r1; ++r) {
      const float* p = src + base + (thb_i64)r * inner;
      float* d = dst + base + (thb_i64)r * inner;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        acc[j] = Op::apply(acc[j], (double)p[j]);
        if (!TOTALS) d[j] = (float)acc[j];
      }
    }
    if (TOTALS) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) carry[cbase + j] = acc[j];
    }
  }
}

// Phase 2 of a chunked scan: the chunk totals of every (outer, inner) position become
// the carries (exclusive scan over the chunks, in chunk order). A block is 32 positions x 8
// lanes; lane k first folds the k-th run of consecutive chunks, the 8 run totals are
// scanned through shared memory, then every lane rewrites its run with the running carry.
template <class Op>
__global__ void __launch_bounds__(THB_SC_THREADS)
thb_scan_carries(double* carry, thb_i64 outer, thb_u32 nchunks, thb_i64 inner) {
  __shared__ double runs[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const thb_u32 per = (nchunks + 7) >> 3;
  const thb_u32 k0 = min(nchunks, ty * per), k1 = min(nchunks, k0 + per);
  const thb_i64 total = outer * inner;
  for (thb_i64 q0 = (thb_i64)blockIdx.x * 32; q0 < total; q0 += (thb_i64)gridDim.x * 32) {
    const thb_i64 q = q0 + tx;
    const bool live = q < total;
    const thb_i64 o = live ? q / inner : 0, i = live ? q - o * inner : 0;
    double* c = carry + o * nchunks * inner + i;
    double tot = Op::identity();
    if (live) {
      thb_u32 k = k0;
      for (; k + 4 <= k1; k += 4) {
        double t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) t[u] = c[(thb_i64)(k + u) * inner];
#pragma unroll
        for (int u = 0; u < 4; ++u) tot = Op::apply(tot, t[u]);
      }
      for (; k < k1; ++k) tot = Op::apply(tot, c[(thb_i64)k * inner]);
    }
    runs[ty][tx] = tot;
    __syncthreads();
    if (live) {
      double run = Op::identity();
      for (int w = 0; w < ty; ++w) run = Op::apply(run, runs[w][tx]);
      for (thb_u32 k = k0; k < k1; ++k) {
        const double t = c[(thb_i64)k * inner];
        c[(thb_i64)k * inner] = run;
        run = Op::apply(run, t);
      }
    }
    __syncthreads();
  }
}

// The same for inner == 1 when a row has many chunks: one block per row scans the chunk
// totals 256 at a time (shuffle scan inside each warp, the 8 warp totals through shared
// memory), so a single long row does not leave one thread walking thousands of chunks.
template <class Op>
__global__ void __launch_bounds__(THB_SC_THREADS)
thb_scan_carries_rows(double* carry, thb_i64 nrows, thb_u32 nchunks) {
  __shared__ double wtot[THB_SC_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (thb_i64 row = blockIdx.x; row < nrows; row += gridDim.x) {
    double* c = carry + row * nchunks;
    double run = Op::identity();
    for (thb_u32 k0 = 0; k0 < nchunks; k0 += THB_SC_THREADS) {
      const thb_u32 k = k0 + threadIdx.x;
      const double t = k < nchunks ? c[k] : Op::identity();
      double incl = t;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const double u = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl = Op::apply(u, incl);
      }
      if (lane == 31) wtot[warp] = incl;
      __syncthreads();
      double before = run;  // everything before this warp's 32 chunks
      for (int w = 0; w < warp; ++w) before = Op::apply(before, wtot[w]);
      double excl = __shfl_up_sync(0xffffffffu, incl, 1);
      if (lane == 0) excl = Op::identity();
      if (k < nchunks) c[k] = Op::apply(before, excl);
#pragma unroll
      for (int w = 0; w < THB_SC_THREADS / 32; ++w) run = Op::apply(run, wtot[w]);
      __syncthreads();
    }
  }
}

// inner == 1: one warp per (row, chunk). Each step takes THB_SC_ROW_UNROLL pieces of
// 32 x VEC consecutive elements: a prefix inside each lane, a shuffle scan of the lane
// totals, then the running value of the row so far.
template <class Op, int VEC, bool TOTALS>
__global__ void __launch_bounds__(THB_SC_THREADS)
thb_scan_rows(float* dst, const float* src, thb_i64 nrows, thb_u32 n, thb_u32 chunk_len, thb_u32 nchunks,
              double* carry) {
  const int lane = threadIdx.x & 31;
  const thb_i64 nwork = nrows * nchunks;
  const thb_i64 warps = (thb_i64)gridDim.x * (THB_SC_THREADS / 32);
  for (thb_i64 w = (thb_i64)blockIdx.x * (THB_SC_THREADS / 32) + (threadIdx.x >> 5); w < nwork; w += warps) {
    const thb_i64 row = w / nchunks;
    const thb_u32 chunk = (thb_u32)(w - row * nchunks);
    const thb_u32 c0 = chunk * chunk_len, c1 = min(n, c0 + chunk_len);
    const float* s = src + row * (thb_i64)n;
    float* d = dst + row * (thb_i64)n;
    double run = (!TOTALS && nchunks > 1) ? carry[w] : Op::identity();
    for (thb_u32 b = c0; b < c1; b += 32 * VEC * THB_SC_ROW_UNROLL) {
      float v[THB_SC_ROW_UNROLL][VEC];
#pragma unroll
      for (int u = 0; u < THB_SC_ROW_UNROLL; ++u) {
        const thb_u32 e = b + (u * 32 + lane) * VEC;
        if (VEC == 4) {
          // c1 - c0 and n are multiples of 4 on this path, so a vector is all in or all out
          float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
          const bool in = e < c1;
          if (in) t = *reinterpret_cast<const float4*>(s + e);
          const float idf = (float)Op::identity();
          v[u][0] = in ? t.x : idf; v[u][1 % VEC] = in ? t.y : idf; v[u][2 % VEC] = in ? t.z : idf; v[u][3 % VEC] = in ? t.w : idf;
        } else {
          v[u][0] = e < c1 ? s[e] : (float)Op::identity();
        }
      }
#pragma unroll
      for (int u = 0; u < THB_SC_ROW_UNROLL; ++u) {
        const thb_u32 e = b + (u * 32 + lane) * VEC;
        double pre[VEC];
        pre[0] = (double)v[u][0];
#pragma unroll
        for (int j = 1; j < VEC; ++j) pre[j] = Op::apply(pre[j - 1], (double)v[u][j]);
        double incl = pre[VEC - 1];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const double t = __shfl_up_sync(0xffffffffu, incl, off);
          if (lane >= off) incl = Op::apply(t, incl);
        }
        double excl = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane == 0) excl = Op::identity();
        const double before = Op::apply(run, excl);
        if (!TOTALS && e < c1) {
          float o4[VEC];
#pragma unroll
          for (int j = 0; j < VEC; ++j) o4[j] = (float)Op::apply(before, pre[j]);
          if (VEC == 4) *reinterpret_cast<float4*>(d + e) = make_float4(o4[0], o4[1 % VEC], o4[2 % VEC], o4[3 % VEC]);
          else d[e] = o4[0];
        }
        run = Op::apply(run, __shfl_sync(0xffffffffu, incl, 31));
      }
    }
    if (TOTALS && lane == 0) carry[w] = run;
  }
}

// ---- renorm -----------------------------------------------------------------
// Row r of data ([rows][size], contiguous) is multiplied by maxnorm / (norm + 1e-7)
// when norm = sumpow[r]^(1/p) exceeds maxnorm, and left untouched (not even read)
// otherwise. One block per piece of THB_RN_PIECE elements of a row.
#define THB_RN_PIECE 8192
static __global__ void __launch_bounds__(THB_SC_THREADS)
thb_renorm_scale(float* data, const float* sumpow, thb_i64 rows, thb_i64 size, float p, float maxnorm,
                 thb_i64 pieces_per_row) {
  const thb_i64 total = rows * pieces_per_row;
  for (thb_i64 w = blockIdx.x; w < total; w += gridDim.x) {
    const thb_i64 row = w / pieces_per_row, piece = w - row * pieces_per_row;
    const float norm = thb_pow(sumpow[row], 1.0f / p);
    if (!(norm > maxnorm)) continue;
    const float f = (float)((double)maxnorm / ((double)norm + 1e-7));
    float* r = data + row * size;
    const thb_i64 e0 = piece * THB_RN_PIECE, e1 = min(size, e0 + (thb_i64)THB_RN_PIECE);
    if (((((thb_u64)(r + e0)) & 15) == 0) && ((e1 - e0) & 3) == 0) {
      float4* r4 = reinterpret_cast<float4*>(r + e0);
      const int nv = (int)((e1 - e0) >> 2);
      for (int i = threadIdx.x; i < nv; i += THB_SC_THREADS) {
        float4 t = r4[i];
        t.x *= f; t.y *= f; t.z *= f; t.w *= f;
        r4[i] = t;
      }
    } else {
      for (thb_i64 i = e0 + threadIdx.x; i < e1; i += THB_SC_THREADS) r[i] *= f;
    }
  }
}

// ---- dist -------------------------------------------------------------------
// Pass 1 of sum |a - b|^p over two contiguous vectors (any alignment: scalar head/tail
// handled by block 0 when the vectors are not both 16-byte aligned).
static __global__ void __launch_bounds__(THB_RA_THREADS, THB_RA_BLOCKS_PER_SM)
thb_dist_pass1(const float* a, const float* b, thb_i64 n, float p, int vec_ok, double* partials) {
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
        const thb_i64 i = base + u * THB_RA_THREADS;
        if (i < nvec) { x[u] = a4[i]; y[u] = b4[i]; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const thb_i64 i = base + u * THB_RA_THREADS;
        if (i < nvec) {
          acc[0] += (double)thb_abs_pow(x[u].x - y[u].x, p);
          acc[1] += (double)thb_abs_pow(x[u].y - y[u].y, p);
          acc[2] += (double)thb_abs_pow(x[u].z - y[u].z, p);
          acc[3] += (double)thb_abs_pow(x[u].w - y[u].w, p);
        }
      }
    }
    if (blockIdx.x == 0) {
      const thb_i64 t = (nvec << 2) + threadIdx.x;
      if (t < n) acc[0] += (double)thb_abs_pow(a[t] - b[t], p);
    }
  } else {
    for (thb_i64 i = (thb_i64)blockIdx.x * THB_RA_THREADS + threadIdx.x; i < n; i += (thb_i64)gridDim.x * THB_RA_THREADS)
      acc[0] += (double)thb_abs_pow(a[i] - b[i], p);
  }
  double r = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  r = thb_block_fold<RedAdd>(r, 0.0, smem);
  if (threadIdx.x == 0) partials[blockIdx.x] = r;
}

// Pass 2: fold of the partials, then the 1/p power.
static __global__ void __launch_bounds__(1024)
thb_dist_pass2(const double* partials, int count, float p, float* out) {
  __shared__ double smem[32];
  double r = 0.0;
  for (int i = threadIdx.x; i < count; i += blockDim.x) r += partials[i];
  r = thb_block_fold<RedAdd>(r, 0.0, smem);
  if (threadIdx.x == 0) out[0] = (float)pow(r, 1.0 / (double)p);
}
