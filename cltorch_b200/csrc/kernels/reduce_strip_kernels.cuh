// Reductions (sums, products, variances; max / min with indices) along a non-innermost
// dimension of a contiguous [outer][n][inner] tensor through the TMA strip pipeline of
// scan_strip_kernels.cuh: a work item is a strip of
// 128 columns x a chunk of rows; persistent CTAs stream their items through 8 stages of
// 32 rows x 512 bytes (128 KB of loads in flight per CTA), one column per consumer thread.
// Compared with one thread per 4 columns issuing its own loads (thb_reduce_dim_noncontig_v4,
// thb_argreduce_cols_v4) this keeps HBM busier: 0.87 -> 0.90-0.95 of the measured copy rate
// on 1 GiB inputs.
//
// Same job as THClTensor_kernel_transformReduceOuterDimIndex
// (reference src/lib/THClTensorMathTransformReduce.cl:17-41).
//
// A `Consumer` holds what one thread carries along its column:
//   begin(geometry, item)   at the start of a work item
//   row(value, row_index, slot, weight)   for every row of the item, in ascending order; slot
//                           is a compile-time constant after unrolling (0..3); weight is the
//                           row's weight when Consumer::kRowWeights (then
//                           Consumer::weight(params, row) says what it is), else unused
//   end()                   result or chunk partial of the column
// Every wait is bounded as in the scan kernel; a wait that gives up writes *status.
#pragma once
#include "scan_strip_kernels.cuh"

#define THB_SS_WRING 16  // slots of the row-weight ring (32 floats each): 2 KB, twice the stages

struct ThbStripGeom {
  thb_u32 n;               // length of the reduced dimension
  thb_i64 inner;           // columns per outer index (row pitch in elements)
  int strips_per_outer, total_strips;
  thb_u32 nchunks, chunk_rows;  // chunk_rows is a multiple of THB_SS_ROWS
  thb_u32 npartials;       // partial results per column: nchunks x HALVES
  thb_u32 nslices;         // outer * inner
};

// HALVES = 1: 4 consumer warps, a thread takes every row of its column. HALVES = 2: 8 consumer
// warps, two threads per column taking the even and the odd rows of each stage and producing
// one partial each (for consumers whose per-row work is a chain of fp64 operations: twice the
// warps hide twice the latency).
template <class Consumer, int HALVES>
__global__ void __launch_bounds__(32 + 128 * HALVES, 1)
thb_strip_reduce(const __grid_constant__ CUtensorMap map_src, ThbStripGeom g, typename Consumer::Params cp, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  uint64_t* bar_full = (uint64_t*)(smem + THB_SS_STAGES * THB_SS_STAGE_BYTES);
  uint64_t* bar_empty = bar_full + THB_SS_STAGES;
  volatile int* abort_flag = (volatile int*)(bar_empty + THB_SS_STAGES);
  volatile int* never_set = abort_flag + 1;
  float* weights = (float*)(smem + THB_SS_STAGES * THB_SS_STAGE_BYTES + 512);  // [stage][row], kRowWeights only

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < THB_SS_STAGES; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_full[s]), 1);
      thb_mbar_init(thb_smem_u32(&bar_empty[s]), 4 * HALVES);  // one arrival per consumer warp
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // item -> (chunk, strip): consecutive CTAs take neighbouring strips of the same rows
  const int total_items = g.total_strips * (int)g.nchunks;

  if (warp == 0) {
    // Producer warp: lane 0 waits for a free stage and issues the TMA load; with row weights
    // (Consumer::kRowWeights) all 32 lanes first put the stage's 32 weights into shared memory, so
    // that the consumers do not load them from global memory once per column.
    long long it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int chunk = item / g.total_strips, strip = item - chunk * g.total_strips;
      const int o = strip / g.strips_per_outer;
      const int c0 = (strip - o * g.strips_per_outer) * THB_SS_COLS;
      const thb_u32 r0 = (thb_u32)chunk * g.chunk_rows, r1 = min(g.n, r0 + g.chunk_rows);
      // Row weights travel through a ring of THB_SS_WRING slots of 32 floats, four stages at a
      // time: the batch written at stage q (q % 4 == 0) was loaded four stages earlier, so the
      // producer never sits out the latency of its own load (once per item excepted).
      // Within a slot the weights of the rows a consumer half takes (half, half + HALVES, ...) are
      // adjacent, so that a consumer reads them as vectors of four.
      const int wpos = (lane % HALVES) * (THB_SS_ROWS / HALVES) + lane / HALVES;
      float batch[4];
      thb_u32 q = 0;  // stage index within the item
      if (Consumer::kRowWeights) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const thb_u32 j = r0 + k * THB_SS_ROWS + lane;
          weights[((it + k) % THB_SS_WRING) * THB_SS_ROWS + wpos] = j < r1 ? Consumer::weight(cp, j) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const thb_u32 j = r0 + (4 + k) * THB_SS_ROWS + lane;
          batch[k] = j < r1 ? Consumer::weight(cp, j) : 0.f;
        }
        __syncwarp();
      }
      for (thb_u32 r = r0; r < r1; r += THB_SS_ROWS, ++it) {
        const int s = (int)(it % THB_SS_STAGES);
        const uint32_t round = (uint32_t)(it / THB_SS_STAGES);
        int free_ok = 1;
        if (lane == 0 && it >= THB_SS_STAGES && !thb_mbar_wait(thb_smem_u32(&bar_empty[s]), (round - 1) & 1, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; if (status) atomicCAS(status, 0, 1); }
          free_ok = 0;
        }
        free_ok = __shfl_sync(0xffffffffu, free_ok, 0);
        if (!free_ok) { ok = false; break; }
        if (Consumer::kRowWeights) {
          if (q > 0 && (q & 3) == 0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) weights[((it + k) % THB_SS_WRING) * THB_SS_ROWS + wpos] = batch[k];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const thb_u32 j = r + (4 + k) * THB_SS_ROWS + lane;
              batch[k] = j < r1 ? Consumer::weight(cp, j) : 0.f;
            }
            __syncwarp();
          }
          ++q;
        }
        if (lane == 0) {
          const uint32_t full = thb_smem_u32(&bar_full[s]);
          thb_mbar_expect_tx(full, THB_SS_STAGE_BYTES);  // releases the weights written above with it
          thb_tma_load_3d(thb_smem_u32(smem + s * THB_SS_STAGE_BYTES), &map_src, full, c0, (int)r, o);
        }
      }
    }
    if (lane == 0 && *abort_flag) {
      // do not leave while copies into this CTA's shared memory are in flight
      for (long long j = (it > THB_SS_STAGES ? it - THB_SS_STAGES : 0); j < it; ++j)
        thb_mbar_wait(thb_smem_u32(&bar_full[j % THB_SS_STAGES]), (uint32_t)(j / THB_SS_STAGES) & 1, never_set);
    }
  } else {
    const int tx = (threadIdx.x - 32) & (THB_SS_COLS - 1);
    const int half = (threadIdx.x - 32) / THB_SS_COLS;  // 0 .. HALVES-1: which rows of a stage
    constexpr int kRows = THB_SS_ROWS / HALVES;
    long long it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int chunk = item / g.total_strips, strip = item - chunk * g.total_strips;
      const int o = strip / g.strips_per_outer;
      const thb_i64 col = (thb_i64)(strip - o * g.strips_per_outer) * THB_SS_COLS + tx;
      const bool live = col < g.inner;
      const thb_u32 r0 = (thb_u32)chunk * g.chunk_rows, r1 = min(g.n, r0 + g.chunk_rows);
      Consumer c;
      c.begin(cp, g, o, col, live, chunk);
      for (thb_u32 rb = r0; rb < r1; rb += THB_SS_ROWS, ++it) {
        const int s = (int)(it % THB_SS_STAGES);
        const uint32_t round = (uint32_t)(it / THB_SS_STAGES);
        bool got = thb_mbar_wait(thb_smem_u32(&bar_full[s]), round & 1, abort_flag);
        if (!got && !*abort_flag) { *abort_flag = 1; if (status) atomicCAS(status, 0, 2); }
        got = __all_sync(0xffffffffu, got);
        if (!got) { ok = false; break; }
        const float* tile = reinterpret_cast<const float*>(smem + s * THB_SS_STAGE_BYTES) + tx + half * THB_SS_COLS;
        float v[kRows];
        float w[Consumer::kRowWeights ? kRows : 1];
#pragma unroll
        for (int k = 0; k < kRows; ++k) v[k] = tile[k * HALVES * THB_SS_COLS];  // rows half, half + HALVES, ...
        if constexpr (Consumer::kRowWeights) {
#pragma unroll
          for (int k4 = 0; k4 < kRows / 4; ++k4) {
            const float4 t = reinterpret_cast<const float4*>(weights + (it % THB_SS_WRING) * THB_SS_ROWS + half * kRows)[k4];
            w[4 * k4 + 0] = t.x; w[4 * k4 + 1] = t.y; w[4 * k4 + 2] = t.z; w[4 * k4 + 3] = t.w;
          }
        }
        __syncwarp();
        if (lane == 0) thb_mbar_arrive(thb_smem_u32(&bar_empty[s]));
        if (rb + THB_SS_ROWS <= r1) {
#pragma unroll
          for (int k = 0; k < kRows; ++k) c.row(v[k], rb + k * HALVES + half, k & 3, w[Consumer::kRowWeights ? k : 0]);
        } else {
#pragma unroll
          for (int k = 0; k < kRows; ++k)
            if (rb + k * HALVES + half < r1) c.row(v[k], rb + k * HALVES + half, k & 3, w[Consumer::kRowWeights ? k : 0]);
        }
      }
      if (ok && live) c.end(cp, g, o, col, chunk * HALVES + half);
    }
  }
  __syncthreads();
}

// ---- consumers ----------------------------------------------------------------

// Sums, products, moments ...: four accumulators per thread (rows 4k + j of the thread's rows into
// accumulator j) because the additions of a column are a chain of dependent fp64 operations.
template <class Mod, class Red>
struct ThbReduceConsumer {
  static constexpr bool kRowWeights = false;
  typedef typename Red::acc_t acc_t;
  struct Params {
    ThbLayout out;       // result of slice s at out.data[thb_offset(out, s)]
    const float* src;    // for operators that want the first element of the slice
    acc_t* partial;      // [npartials][nslices] when npartials > 1
    float init, mparam;
  };
  acc_t acc[4];
  float k0, mparam;
  __device__ __forceinline__ void begin(const Params& p, const ThbStripGeom& g, int o, thb_i64 col, bool live, int) {
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = (acc_t)p.init;
    mparam = p.mparam;
    k0 = (Mod::kFirst && live) ? p.src[(thb_i64)o * g.n * g.inner + col] : 0.f;
  }
  static __device__ __forceinline__ float weight(const Params&, thb_u32) { return 0.f; }
  __device__ __forceinline__ void row(float v, thb_u32, int slot, float) {
    acc[slot] = Red::apply(acc[slot], Mod::apply(v, mparam, k0));
  }
  __device__ __forceinline__ void end(const Params& p, const ThbStripGeom& g, int o, thb_i64 col, int part) {
    const acc_t a = Red::apply(Red::apply(acc[0], acc[1]), Red::apply(acc[2], acc[3]));
    const thb_u32 s = (thb_u32)((thb_i64)o * g.inner + col);
    if (g.npartials == 1) p.out.data[thb_offset(p.out, s)] = Red::result(a, (float)g.n);
    else p.partial[(thb_u64)part * g.nslices + s] = a;
  }
};

template <bool IS_MAX>
struct ThbArgConsumer {
  static constexpr bool kRowWeights = false;
  struct Params {
    float* values;   // contiguous [outer][1][inner]
    float* indices;
    float* pval;     // [nchunks][nslices] when nchunks > 1
    int* pidx;
  };
  float best;
  int idx;
  __device__ __forceinline__ void begin(const Params&, const ThbStripGeom&, int, thb_i64, bool, int) {
    best = ThbArg<IS_MAX>::start();
    idx = -1;
  }
  static __device__ __forceinline__ float weight(const Params&, thb_u32) { return 0.f; }
  __device__ __forceinline__ void row(float v, thb_u32 r, int, float) {
    if (ThbArg<IS_MAX>::strictly(v, best)) { best = v; idx = (int)r; }
  }
  __device__ __forceinline__ void end(const Params& p, const ThbStripGeom& g, int o, thb_i64 col, int chunk) {
    const thb_u64 s = (thb_u64)((thb_i64)o * g.inner + col);
    if (g.npartials == 1) {
      p.values[s] = best;
      p.indices[s] = (float)(idx < 0 ? -1 : idx + 1);
    } else {
      p.pval[(thb_u64)chunk * g.nslices + s] = best;
      p.pidx[(thb_u64)chunk * g.nslices + s] = idx;
    }
  }
};
