// Pointwise apply kernels for sm_100a.
//
// This header is FREESTANDING (no #include): the same text is compiled by nvcc
// for the built-in operators and handed to NVRTC at run time for user
// expressions (apply/map/map2), so both run through identical launch code.
//
// What it replaces: the OpenCL template THClTensor_pointwiseApplyD
// (reference src/lib/THClApply.cl:47-102), which maps one work-item to one
// element and recomputes `offset + sum((lin % size_d) * stride_d)` per operand.
//
// An operator is a struct with
//   static __device__ void apply(float* out, const float* in1, const float* in2,
//                                float val1, float val2,
//                                const float* pointTensor1, const float* pointTensor2);
//   static constexpr bool kReadsOut;   // false: `out` is write-only, its load is skipped
// The parameter names are the ones the reference's operator strings use
// (src/lib/THClTensorMathPointwise.h, src/lib/THClApply.cl:33-45), so those
// strings paste in unchanged.
//
// Four kernels:
//   thb_apply_contig   every operand is one contiguous run: 128-bit loads and
//                      stores, 4 vectors in flight per thread, 64-bit counts.
//   thb_apply_rows2d   the same R x C matrix in every operand with unit stride
//                      along C (column-narrowed views): 128-bit along the rows.
//   thb_apply_strided  any collapsed layout up to 25 dims, 32-bit index math
//                      with multiply-shift division instead of % and /.
//   thb_apply_tile2d   operands are the same logical R x C matrix, each either
//                      row-major-like (unit stride along C) or column-major-like
//                      (unit stride along R, e.g. a transpose view): the
//                      column-major ones go through a padded shared-memory tile
//                      so that every global access is coalesced.
#pragma once

typedef long long thb_i64;
typedef unsigned long long thb_u64;
typedef unsigned int thb_u32;

#define THB_MAX_DIMS 25  // MAX_CLTORCH_DIMS, reference src/lib/THClReduceApplyUtils.h:19

// Collapsed layout of one operand (what TensorInfo<uint32> holds in the
// reference, src/lib/THClReduceApplyUtils.h:43-66) plus the constants of an
// exact unsigned division by each size.
struct ThbLayout {
  float* data;  // element (0,...,0) of the view: storage base + storageOffset
  int dims;
  thb_u32 size[THB_MAX_DIMS];
  thb_u32 stride[THB_MAX_DIMS];
  thb_u32 magic[THB_MAX_DIMS];  // see thb_fastdiv
  thb_u32 shift[THB_MAX_DIMS];  // sh1 | (sh2 << 8)
};

// floor(n / d) for any 32-bit n: q = (t + ((n - t) >> sh1)) >> sh2 with
// t = umulhi(magic, n) (division by an invariant integer, Granlund & Montgomery).
__device__ __forceinline__ thb_u32 thb_fastdiv(thb_u32 n, thb_u32 magic, thb_u32 shift) {
  thb_u32 t = __umulhi(magic, n);
  return (t + ((n - t) >> (shift & 0xffu))) >> (shift >> 8);
}

__device__ __forceinline__ thb_u32 thb_offset(const ThbLayout& L, thb_u32 lin) {
  // Row-major decomposition of the linear index in the operand's own shape,
  // innermost dimension first (reference src/lib/THClApply.cl:70-85).
  if (L.dims == 1) return lin * L.stride[0];
  thb_u32 off = 0;
  for (int d = L.dims - 1; d > 0; --d) {
    thb_u32 q = thb_fastdiv(lin, L.magic[d], L.shift[d]);
    off += (lin - q * L.size[d]) * L.stride[d];
    lin = q;
  }
  return off + lin * L.stride[0];
}

struct ThbScalars {
  float val1, val2;
  const float* pointTensor1;  // device-resident 1-float results of a reduceAll
  const float* pointTensor2;
};

// ---------------------------------------------------------------------------
// Contiguous operands.
// `head` (0..3) elements come before the first 16-byte boundary, which all
// operands share; block 0 handles them and the (n - head) % 4 trailing ones.
// ---------------------------------------------------------------------------
#define THB_CONTIG_THREADS 256
#define THB_CONTIG_UNROLL 4

// For kernels launched with programmatic stream serialisation (their blocks may become resident
// while the previous kernel of the stream drains): wait until that kernel has completed and its
// writes are visible, then let the next kernel's blocks be placed in turn. Without the launch
// attribute both instructions do nothing.
__device__ __forceinline__ void thb_grid_dependency_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <class Op, int NT>
__global__ void __launch_bounds__(THB_CONTIG_THREADS)
thb_apply_contig(float* a, const float* b, const float* c, thb_i64 n, int head, ThbScalars s) {
  thb_grid_dependency_sync();
  float p1 = 0.f, p2 = 0.f;
  if (s.pointTensor1) p1 = *s.pointTensor1;
  if (s.pointTensor2) p2 = *s.pointTensor2;

  // bit 8 of `head`: walk the batches from the last to the first (the host asks for it when the end of the
  // operands is what the previous kernel left in L2)
  const bool reverse = (head & 256) != 0;
  head &= 255;
  const thb_i64 nvec = (n - head) >> 2;
  float4* a4 = reinterpret_cast<float4*>(a + head);
  const float4* b4 = reinterpret_cast<const float4*>(b + head);
  const float4* c4 = reinterpret_cast<const float4*>(c + head);

  constexpr int kBatch = THB_CONTIG_THREADS * THB_CONTIG_UNROLL;
  const thb_i64 nbatch = (nvec + kBatch - 1) / kBatch;
  for (thb_i64 batch = blockIdx.x; batch < nbatch; batch += gridDim.x) {
    const thb_i64 base = (reverse ? nbatch - 1 - batch : batch) * kBatch + threadIdx.x;
    float4 va[THB_CONTIG_UNROLL], vb[THB_CONTIG_UNROLL], vc[THB_CONTIG_UNROLL];
#pragma unroll
    for (int u = 0; u < THB_CONTIG_UNROLL; ++u) {
      thb_i64 i = base + u * THB_CONTIG_THREADS;
      if (i < nvec) {
        if (Op::kReadsOut) va[u] = a4[i];
        if (NT >= 2) vb[u] = b4[i];
        if (NT >= 3) vc[u] = c4[i];
      }
    }
#pragma unroll
    for (int u = 0; u < THB_CONTIG_UNROLL; ++u) {
      thb_i64 i = base + u * THB_CONTIG_THREADS;
      if (i < nvec) {
        Op::apply(&va[u].x, &vb[u].x, &vc[u].x, s.val1, s.val2, &p1, &p2);
        Op::apply(&va[u].y, &vb[u].y, &vc[u].y, s.val1, s.val2, &p1, &p2);
        Op::apply(&va[u].z, &vb[u].z, &vc[u].z, s.val1, s.val2, &p1, &p2);
        Op::apply(&va[u].w, &vb[u].w, &vc[u].w, s.val1, s.val2, &p1, &p2);
        a4[i] = va[u];
      }
    }
  }

  if (blockIdx.x == 0) {
    // ragged ends: at most 3 leading and 3 trailing elements
    const thb_i64 tail0 = head + (nvec << 2);
    const int ntail = (int)(n - tail0);
    int t = threadIdx.x;
    thb_i64 i = -1;
    if (t < head) i = t;
    else if (t - head < ntail) i = tail0 + (t - head);
    if (i >= 0) {
      float o = 0.f, x = 0.f, y = 0.f;
      if (Op::kReadsOut) o = a[i];
      if (NT >= 2) x = b[i];
      if (NT >= 3) y = c[i];
      Op::apply(&o, &x, &y, s.val1, s.val2, &p1, &p2);
      a[i] = o;
    }
  }
}

// ---------------------------------------------------------------------------
// Any strided layout, 32-bit index math (n < 2^32).
// ---------------------------------------------------------------------------
#define THB_STRIDED_THREADS 256
#define THB_STRIDED_UNROLL 4

template <class Op, int NT>
__global__ void __launch_bounds__(THB_STRIDED_THREADS)
thb_apply_strided(ThbLayout A, ThbLayout B, ThbLayout C, thb_u64 n, ThbScalars s) {
  thb_grid_dependency_sync();
  float p1 = 0.f, p2 = 0.f;
  if (s.pointTensor1) p1 = *s.pointTensor1;
  if (s.pointTensor2) p2 = *s.pointTensor2;

  const thb_u64 step = (thb_u64)gridDim.x * (THB_STRIDED_THREADS * THB_STRIDED_UNROLL);
  for (thb_u64 base = (thb_u64)blockIdx.x * (THB_STRIDED_THREADS * THB_STRIDED_UNROLL) + threadIdx.x;
       base < n; base += step) {
    float o[THB_STRIDED_UNROLL], x[THB_STRIDED_UNROLL], y[THB_STRIDED_UNROLL];
    thb_u32 oa[THB_STRIDED_UNROLL];
#pragma unroll
    for (int u = 0; u < THB_STRIDED_UNROLL; ++u) {
      thb_u64 i = base + (thb_u64)u * THB_STRIDED_THREADS;
      o[u] = x[u] = y[u] = 0.f;
      if (i < n) {
        thb_u32 lin = (thb_u32)i;
        oa[u] = thb_offset(A, lin);
        if (Op::kReadsOut) o[u] = A.data[oa[u]];
        if (NT >= 2) x[u] = B.data[thb_offset(B, lin)];
        if (NT >= 3) y[u] = C.data[thb_offset(C, lin)];
      }
    }
#pragma unroll
    for (int u = 0; u < THB_STRIDED_UNROLL; ++u) {
      thb_u64 i = base + (thb_u64)u * THB_STRIDED_THREADS;
      if (i < n) {
        Op::apply(&o[u], &x[u], &y[u], s.val1, s.val2, &p1, &p2);
        A.data[oa[u]] = o[u];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Same logical R x C matrix in every operand, unit stride along C and any row
// stride (column-narrowed views, or a contiguous tensor seen as R x C): float4
// along the rows, one division per vector shared by all operands. Needs
// C % 4 == 0, 16-byte aligned row starts, and fewer than 2^32 vectors.
// ---------------------------------------------------------------------------
struct ThbRows2d {
  float* data[3];
  thb_i64 row_stride[3];  // elements
  thb_u32 cvec;           // C / 4
  thb_u32 magic, shift;   // division by cvec
  thb_u64 nvec;           // R * cvec
};

template <class Op, int NT>
__global__ void __launch_bounds__(THB_CONTIG_THREADS)
thb_apply_rows2d(ThbRows2d P, ThbScalars s) {
  thb_grid_dependency_sync();
  float p1 = 0.f, p2 = 0.f;
  if (s.pointTensor1) p1 = *s.pointTensor1;
  if (s.pointTensor2) p2 = *s.pointTensor2;
  const thb_u64 step = (thb_u64)gridDim.x * (THB_CONTIG_THREADS * THB_CONTIG_UNROLL);
  for (thb_u64 base = (thb_u64)blockIdx.x * (THB_CONTIG_THREADS * THB_CONTIG_UNROLL) + threadIdx.x;
       base < P.nvec; base += step) {
    float4 va[THB_CONTIG_UNROLL], vb[THB_CONTIG_UNROLL], vc[THB_CONTIG_UNROLL];
    float4* pa[THB_CONTIG_UNROLL];
#pragma unroll
    for (int u = 0; u < THB_CONTIG_UNROLL; ++u) {
      const thb_u64 i = base + (thb_u64)u * THB_CONTIG_THREADS;
      if (i < P.nvec) {
        const thb_u32 r = thb_fastdiv((thb_u32)i, P.magic, P.shift);
        const thb_u32 c = ((thb_u32)i - r * P.cvec) << 2;
        pa[u] = reinterpret_cast<float4*>(P.data[0] + (thb_i64)r * P.row_stride[0] + c);
        if (Op::kReadsOut) va[u] = *pa[u];
        if (NT >= 2) vb[u] = *reinterpret_cast<const float4*>(P.data[1] + (thb_i64)r * P.row_stride[1] + c);
        if (NT >= 3) vc[u] = *reinterpret_cast<const float4*>(P.data[2] + (thb_i64)r * P.row_stride[2] + c);
      }
    }
#pragma unroll
    for (int u = 0; u < THB_CONTIG_UNROLL; ++u) {
      const thb_u64 i = base + (thb_u64)u * THB_CONTIG_THREADS;
      if (i < P.nvec) {
        Op::apply(&va[u].x, &vb[u].x, &vc[u].x, s.val1, s.val2, &p1, &p2);
        Op::apply(&va[u].y, &vb[u].y, &vc[u].y, s.val1, s.val2, &p1, &p2);
        Op::apply(&va[u].z, &vb[u].z, &vc[u].z, s.val1, s.val2, &p1, &p2);
        Op::apply(&va[u].w, &vb[u].w, &vc[u].w, s.val1, s.val2, &p1, &p2);
        *pa[u] = va[u];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Same logical R x C matrix in every operand; element (r, c) of operand t sits
// at data_t[r * sr_t + c * sc_t]. colmajor bit t set: sr_t == 1 (coalesce
// along r); clear: sc_t == 1 (coalesce along c).
// Tile 32 x 32, block 32 x 8; tiles are enumerated by a 1-D grid.
// ---------------------------------------------------------------------------
#define THB_TILE 32
#define THB_TILE_ROWS 8

struct ThbTile2d {
  float* data[3];
  thb_i64 sr[3];
  thb_i64 sc[3];
  thb_u32 R, C;
  thb_u32 tilesC;   // ceil(C / 32)
  thb_u32 ntiles;   // ceil(R / 32) * tilesC
  int colmajor;     // bit t: operand t is column-major-like
};

template <class Op, int NT>
__global__ void __launch_bounds__(THB_TILE * THB_TILE_ROWS)
thb_apply_tile2d(ThbTile2d P, ThbScalars s) {
  __shared__ float tile[3][THB_TILE][THB_TILE + 1];
  thb_grid_dependency_sync();
  float p1 = 0.f, p2 = 0.f;
  if (s.pointTensor1) p1 = *s.pointTensor1;
  if (s.pointTensor2) p2 = *s.pointTensor2;

  const int tx = threadIdx.x, ty = threadIdx.y;
  for (thb_u32 t = blockIdx.x; t < P.ntiles; t += gridDim.x) {
    const thb_u32 r0 = (t / P.tilesC) * THB_TILE;
    const thb_u32 c0 = (t % P.tilesC) * THB_TILE;

    // stage column-major-like operands: thread (tx, ty+8k) reads element
    // (r0 + tx, c0 + ty + 8k), unit stride along tx
#pragma unroll
    for (int q = 0; q < NT; ++q) {
      if (((P.colmajor >> q) & 1) && (q > 0 || Op::kReadsOut)) {
#pragma unroll
        for (int k = 0; k < THB_TILE; k += THB_TILE_ROWS) {
          thb_u32 r = r0 + tx, c = c0 + ty + k;
          if (r < P.R && c < P.C)
            tile[q][ty + k][tx] = P.data[q][(thb_i64)r * P.sr[q] + (thb_i64)c * P.sc[q]];
        }
      }
    }
    __syncthreads();

    float v[3][THB_TILE / THB_TILE_ROWS];
#pragma unroll
    for (int k = 0; k < THB_TILE / THB_TILE_ROWS; ++k) {
      const thb_u32 r = r0 + ty + k * THB_TILE_ROWS, c = c0 + tx;
      const bool in = (r < P.R && c < P.C);
#pragma unroll
      for (int q = 0; q < NT; ++q) {
        v[q][k] = 0.f;
        if (in && (q > 0 || Op::kReadsOut)) {
          if ((P.colmajor >> q) & 1) v[q][k] = tile[q][tx][ty + k * THB_TILE_ROWS];
          else v[q][k] = P.data[q][(thb_i64)r * P.sr[q] + (thb_i64)c * P.sc[q]];
        }
      }
      if (in) {
        Op::apply(&v[0][k], &v[NT >= 2 ? 1 : 0][k], &v[NT >= 3 ? 2 : 0][k], s.val1, s.val2, &p1, &p2);
        if (!(P.colmajor & 1)) P.data[0][(thb_i64)r * P.sr[0] + (thb_i64)c * P.sc[0]] = v[0][k];
      }
    }

    if (P.colmajor & 1) {
      __syncthreads();  // everyone has taken its inputs out of tile[0]
#pragma unroll
      for (int k = 0; k < THB_TILE / THB_TILE_ROWS; ++k)
        tile[0][tx][ty + k * THB_TILE_ROWS] = v[0][k];
      __syncthreads();
#pragma unroll
      for (int k = 0; k < THB_TILE; k += THB_TILE_ROWS) {
        thb_u32 r = r0 + tx, c = c0 + ty + k;
        if (r < P.R && c < P.C)
          P.data[0][(thb_i64)r * P.sr[0] + (thb_i64)c * P.sc[0]] = tile[0][ty + k][tx];
      }
    }
    __syncthreads();  // tiles are reused by the next iteration
  }
}

// ---------------------------------------------------------------------------
// The same job with 128-bit global accesses on both sides: tiles of 64 rows x
// 32 columns, 256 threads. A column-major-like operand is read as float4 along r
// (16 threads cover the 64 rows of one column: 256 contiguous bytes), kept in
// shared memory as tile[c][r], and picked up per element by the row-major
// mapping, in which a thread owns 4 consecutive columns of one row. Needs every
// operand 16-byte aligned, row-major ones with C % 4 == 0 and a row stride that
// is a multiple of 4, column-major ones with R % 4 == 0 and a column stride that
// is a multiple of 4; the host falls back to thb_apply_tile2d otherwise.
// ---------------------------------------------------------------------------
#define THB_T4_R 64
#define THB_T4_C 32
#define THB_T4_PITCH 66  // 66 % 32 == 2: the per-element reads below are at most 2-way bank conflicts

template <class Op, int NT>
__global__ void __launch_bounds__(256)
thb_apply_tile2d_v4(ThbTile2d P, ThbScalars s) {
  __shared__ float tile[3][THB_T4_C][THB_T4_PITCH];
  thb_grid_dependency_sync();
  float p1 = 0.f, p2 = 0.f;
  if (s.pointTensor1) p1 = *s.pointTensor1;
  if (s.pointTensor2) p2 = *s.pointTensor2;

  const int tid = threadIdx.x;
  const int cr = tid & 15, cc = tid >> 4;  // column-major mapping: rows 4cr..4cr+3 of columns cc, cc+16
  const int rc = tid & 7, rr = tid >> 3;   // row-major mapping: columns 4rc..4rc+3 of rows rr, rr+32
  for (thb_u32 t = blockIdx.x; t < P.ntiles; t += gridDim.x) {
    const thb_u32 r0 = (t / P.tilesC) * THB_T4_R;
    const thb_u32 c0 = (t % P.tilesC) * THB_T4_C;

#pragma unroll
    for (int q = 0; q < NT; ++q) {
      if (((P.colmajor >> q) & 1) && (q > 0 || Op::kReadsOut)) {
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const thb_u32 r = r0 + 4 * cr, c = c0 + cc + 16 * pass;
          if (r < P.R && c < P.C) {
            const float4 v = *reinterpret_cast<const float4*>(P.data[q] + r + (thb_i64)c * P.sc[q]);
            float2* dst = reinterpret_cast<float2*>(&tile[q][cc + 16 * pass][4 * cr]);
            dst[0] = make_float2(v.x, v.y);
            dst[1] = make_float2(v.z, v.w);
          }
        }
      }
    }
    __syncthreads();

    float4 v[3][2];
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const thb_u32 r = r0 + rr + 32 * pass, c = c0 + 4 * rc;
      const bool in = (r < P.R && c < P.C);
#pragma unroll
      for (int q = 0; q < NT; ++q) {
        v[q][pass] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in && (q > 0 || Op::kReadsOut)) {
          if ((P.colmajor >> q) & 1) {
            v[q][pass].x = tile[q][4 * rc + 0][rr + 32 * pass];
            v[q][pass].y = tile[q][4 * rc + 1][rr + 32 * pass];
            v[q][pass].z = tile[q][4 * rc + 2][rr + 32 * pass];
            v[q][pass].w = tile[q][4 * rc + 3][rr + 32 * pass];
          } else {
            v[q][pass] = *reinterpret_cast<const float4*>(P.data[q] + (thb_i64)r * P.sr[q] + c);
          }
        }
      }
      if (in) {
        float4& o = v[0][pass];
        const float4& x = v[NT >= 2 ? 1 : 0][pass];
        const float4& y = v[NT >= 3 ? 2 : 0][pass];
        Op::apply(&o.x, &x.x, &y.x, s.val1, s.val2, &p1, &p2);
        Op::apply(&o.y, &x.y, &y.y, s.val1, s.val2, &p1, &p2);
        Op::apply(&o.z, &x.z, &y.z, s.val1, s.val2, &p1, &p2);
        Op::apply(&o.w, &x.w, &y.w, s.val1, s.val2, &p1, &p2);
        if (!(P.colmajor & 1)) *reinterpret_cast<float4*>(P.data[0] + (thb_i64)r * P.sr[0] + c) = o;
      }
    }

    if (P.colmajor & 1) {
      __syncthreads();  // everyone has taken its inputs out of tile[0]
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        tile[0][4 * rc + 0][rr + 32 * pass] = v[0][pass].x;
        tile[0][4 * rc + 1][rr + 32 * pass] = v[0][pass].y;
        tile[0][4 * rc + 2][rr + 32 * pass] = v[0][pass].z;
        tile[0][4 * rc + 3][rr + 32 * pass] = v[0][pass].w;
      }
      __syncthreads();
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const thb_u32 r = r0 + 4 * cr, c = c0 + cc + 16 * pass;
        if (r < P.R && c < P.C) {
          const float2* src = reinterpret_cast<const float2*>(&tile[0][cc + 16 * pass][4 * cr]);
          const float2 lo = src[0], hi = src[1];
          *reinterpret_cast<float4*>(P.data[0] + r + (thb_i64)c * P.sc[0]) = make_float4(lo.x, lo.y, hi.x, hi.y);
        }
      }
    }
    __syncthreads();  // tiles are reused by the next iteration
  }
}

// ---------------------------------------------------------------------------
// Whether a kernel must load *out before running an operator body. It need not
// only when the body is ONE unconditional assignment to *out: the text begins
// with "*out" or "(*out)" followed by a plain '=', "*out" occurs nowhere else,
// and there is no second statement and no block (no ';' before the end, no
// '{'). Anything else - "if (...) *out = ...", a loop, "*out += ..." - may
// leave an element as it was or read it, so the old value has to be there.
// ---------------------------------------------------------------------------
__host__ __device__ constexpr bool thb_is_ident_char(char c) {
  return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '_';
}
__host__ __device__ constexpr bool thb_body_reads_out(const char* s) {
  int count = 0;
  for (int i = 0; s[i]; ++i) {
    if (s[i] == '*' && s[i + 1] == 'o' && s[i + 2] == 'u' && s[i + 3] == 't' && !thb_is_ident_char(s[i + 4])) ++count;
    if (s[i] == '{') return true;
    if (s[i] == ';') {  // only white space may follow the one statement
      int j = i + 1;
      while (s[j] == ' ' || s[j] == '\t' || s[j] == '\n' || s[j] == ';') ++j;
      if (s[j]) return true;
    }
  }
  if (count != 1) return true;
  int i = 0;
  while (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '(') ++i;
  if (!(s[i] == '*' && s[i + 1] == 'o' && s[i + 2] == 'u' && s[i + 3] == 't' && !thb_is_ident_char(s[i + 4]))) return true;
  i += 4;
  while (s[i] == ' ' || s[i] == ')') ++i;
  return !(s[i] == '=' && s[i + 1] != '=');
}

// OpenCL spellings that the reference's operator strings use and CUDA lacks.
__device__ __forceinline__ float powr(float x, float y) { return powf(x, y); }
