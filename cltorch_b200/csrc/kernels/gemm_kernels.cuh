// fp32 GEMM on the 5th-generation tensor cores (tcgen05, sm_100a) with fp32
// accuracy from three TF32 products.
//
//   C(m x n, column-major) = alpha * A' * B'^T + beta * C
//
// Each fp32 operand x is split as x = hi + lo with hi = tf32(x) (round to
// nearest, low 13 mantissa bits zero) and lo = x - hi (exact in fp32). The
// product is accumulated in fp32 in tensor memory as
//   lo_a*hi_b + hi_a*lo_b + hi_a*hi_b
// per 8-deep k step; lo_a*lo_b (relative size 2^-22) is dropped.
//
// Two kernels:
//  thb_gemm_split   reads op(A) (or op(B)) once and writes hi and lo as
//                   row-major [rows][Kp] matrices ("K-major"), Kp = K rounded
//                   up to 32 and zero-filled, so that the GEMM kernel needs a
//                   single operand layout whatever transa/transb were.
//  thb_gemm_3xtf32  persistent, one CTA per SM, 128 x 256 output tiles. Warp 0
//                   lane 0 issues TMA loads (cp.async.bulk.tensor, swizzled, no
//                   multicast) of the four operand tiles of a k block into a
//                   shared-memory ring; warp 1 lane 0 issues
//                   tcgen05.mma.kind::tf32 (M=128, N=256, K=8), three per k
//                   step, into one of two 128-lane x 256-column TMEM
//                   accumulators and commits to mbarriers; warps 2-9 read the
//                   other accumulator with tcgen05.ld (each warp its 32 TMEM lanes
//                   and half of the columns) and write C with coalesced stores
//                   while the next tile's k loop runs; the old C of the next
//                   32 columns is already in flight while a block is stored.
//
// Every wait is bounded: after THB_GEMM_WAIT_LIMIT_NS a waiter records a
// code in *status, raises the CTA's abort flag and everybody falls through to
// the common exit, where tensor memory is released.
#pragma once

#include "tma_pipeline.cuh"

#define THB_GEMM_BM 128
// threads of a CTA: warp 0 TMA, warp 1 MMA issuer, then EW (4 or 8) epilogue warps
#define THB_GEMM_THREADS(EW) (64 + 32 * (EW))
#define THB_GEMM_GROUP_M 16

// Shared-memory budget of one configuration: tile width BN (256, or 128 for problems
// with too few 128 x 256 tiles to fill the GPU), k-block depth BK (32 = 128-byte
// swizzle, 16 = 64-byte swizzle) and ring length STAGES.
template <int BN, int BK, int STAGES>
struct ThbGemmCfg {
  static constexpr int kTileA = THB_GEMM_BM * BK * 4;
  static constexpr int kTileB = BN * BK * 4;
  static constexpr int kTmemCols = 2 * BN;  // two 128 x BN fp32 accumulators
  static constexpr int kStage = 2 * kTileA + 2 * kTileB;  // A_hi, A_lo, B_hi, B_lo
  static constexpr int kSmem = STAGES * kStage + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// ---- operand split ----------------------------------------------------------
// src element (r, k) is at src[r * sr + k * sk]; TRANS selects which of the two
// is the unit-stride direction (false: sk == 1, true: sr == 1).
__device__ __forceinline__ float thb_round_tf32(float x) {
  uint32_t h;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  return __uint_as_float(h);
}

template <bool TRANS>
__global__ void __launch_bounds__(256)
thb_gemm_split(const float* __restrict__ src, long long sr, long long sk, long long batch_stride_src,
               float* __restrict__ dst, int rows, int K, int Kp) {
  // dst: [batch][2][rows][Kp], part 0 = hi, part 1 = lo
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  const float* s = src + (long long)b * batch_stride_src;
  float* hi = dst + ((long long)b * 2 + 0) * rows * (long long)Kp;
  float* lo = dst + ((long long)b * 2 + 1) * rows * (long long)Kp;
  const int k0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  if (TRANS) {
    // unit stride along r: read (r0 + tx, k0 + ty + 8j), transpose through smem
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      int r = r0 + tx, k = k0 + ty + j;
      tile[ty + j][tx] = (r < rows && k < K) ? s[(long long)r * sr + (long long)k * sk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      int r = r0 + ty + j, k = k0 + tx;
      if (r < rows && k < Kp) {
        float x = tile[tx][ty + j];
        const float h = thb_round_tf32(x);
        hi[(long long)r * Kp + k] = h;
        lo[(long long)r * Kp + k] = x - h;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      int r = r0 + ty + j, k = k0 + tx;
      if (r < rows && k < Kp) {
        float x = (k < K) ? s[(long long)r * sr + (long long)k * sk] : 0.f;
        const float h = thb_round_tf32(x);
        hi[(long long)r * Kp + k] = h;
        lo[(long long)r * Kp + k] = x - h;
      }
    }
  }
}

// The same split for a K-major source (unit stride along k) whose rows start on 16-byte boundaries:
// one thread takes 4 consecutive k of one row with 128-bit accesses. Block = 32 x 8 threads = 128 k x 8 rows.
static __global__ void __launch_bounds__(256)
thb_gemm_split_rows_v4(const float* __restrict__ src, long long sr, long long batch_stride_src, float* __restrict__ dst,
                       int rows, int K, int Kp) {
  const int b = blockIdx.z;
  const int k = (blockIdx.x * 32 + (threadIdx.x & 31)) * 4;
  const int r = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (r >= rows || k >= Kp) return;
  const float* s = src + (long long)b * batch_stride_src + (long long)r * sr + k;
  float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
  if (k + 3 < K) {
    x = *reinterpret_cast<const float4*>(s);
  } else {
    if (k < K) x.x = s[0];
    if (k + 1 < K) x.y = s[1];
    if (k + 2 < K) x.z = s[2];
  }
  float4 h;
  h.x = thb_round_tf32(x.x); h.y = thb_round_tf32(x.y); h.z = thb_round_tf32(x.z); h.w = thb_round_tf32(x.w);
  float* hi = dst + ((long long)b * 2 + 0) * rows * (long long)Kp + (long long)r * Kp + k;
  float* lo = dst + ((long long)b * 2 + 1) * rows * (long long)Kp + (long long)r * Kp + k;
  *reinterpret_cast<float4*>(hi) = h;
  *reinterpret_cast<float4*>(lo) = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
}

// ---- PTX helpers (mbarrier and TMA ones are in tma_pipeline.cuh) ------------
// Shared-memory matrix descriptor of a K-major tile whose rows are one swizzle
// span long: BK = 32 floats -> 128-byte swizzle (8-row groups 1024 bytes apart),
// BK = 16 floats -> 64-byte swizzle (8-row groups 512 bytes apart).
template <int BK>
__device__ __forceinline__ uint64_t thb_umma_desc(uint32_t smem_addr) {
  constexpr uint64_t kSbo = (BK == 32) ? 1024 : 512;
  constexpr uint64_t kLayout = (BK == 32) ? 2 : 4;  // 2 = SWIZZLE_128B, 4 = SWIZZLE_64B
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (kSbo >> 4) << 32;                        // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                        // descriptor version of sm_100
  d |= kLayout << 61;
  return d;
}
// Instruction descriptor of tcgen05.mma.kind::tf32: fp32 accumulate, TF32 A and
// B, both K-major, N at bits [17,23) in units of 8, M at bits [24,29) in units of 16.
__device__ __forceinline__ uint32_t thb_umma_idesc_tf32(int M, int N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void thb_umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void thb_umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct ThbGemmParams {
  float* c;
  long long ldc, batch_stride_c;
  int m, n, kblocks;
  float alpha, beta;
  int tiles_m, tiles_n, batch;
  int* status;  // 0 = fine; otherwise the code of the first wait that gave up
  // split-K: work item w = (tile, split); split s takes k blocks [s * kb_per_split, ...) and
  // stores its raw accumulators to partial[s][batch][n][m] (leading dimension m) for
  // thb_gemm_splitk_fixup. splits == 1: results go straight to C.
  int splits, kb_per_split;
  float* partial;
  long long partial_split_stride;
};

// tile index -> (batch, tile_m, tile_n): within a batch, THB_GEMM_GROUP_M row tiles
// share their B tiles in L2
#define THB_GEMM_TILE_COORDS(work)                                          \
const int split = (work) % p.splits;                                      \
const int tile_ = (work) / p.splits;                                      \
const int kb_begin = split * p.kb_per_split;                              \
const int kb_end = min(p.kblocks, kb_begin + p.kb_per_split);             \
const int batch = tile_ / tiles_per_batch;                                \
const int rem_ = tile_ % tiles_per_batch;                                 \
const int first_m_ = (rem_ / group_sz) * THB_GEMM_GROUP_M;                \
const int gm_ = min(THB_GEMM_GROUP_M, p.tiles_m - first_m_);              \
const int tile_m = first_m_ + (rem_ % group_sz) % gm_;                    \
const int tile_n = (rem_ % group_sz) / gm_;


// ---- epilogue, shared by the GEMM kernels: run by warps 2 .. 2+EW-1 of the CTA. Warp w reads
// TMEM lanes 32*(w%4) .. +31 (the lanes a warp may touch); with 8 warps, warps 2-5 take the first
// half of the tile's columns and warps 6-9 the second half.
// NACC = number of TMEM accumulators the kernel alternates between (tile t uses accumulator t % NACC).
// PAIR: the CTA is one of a cluster of two that work on one 256-row tile together (p.tiles_m counts
// those double tiles): work items are taken per cluster, this CTA owns the rows of its rank's half, and
// "accumulator free" is signalled to the barrier of the cluster's first CTA, whose thread issues the MMAs.
template <int BN, int EW, bool PREFETCH_C, int NACC = 2, bool PAIR = false>
__device__ __forceinline__ void thb_gemm_epilogue_loop(const ThbGemmParams& p, const uint32_t tmem_base,
                                                       uint64_t* bar_acc_full, uint64_t* bar_acc_empty,
                                                       volatile int* abort_flag) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch * p.splits;
  const int group_sz = THB_GEMM_GROUP_M * p.tiles_n;
  const int work_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int work_stride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int pair_rank = PAIR ? (int)(blockIdx.x & 1) : 0;
  // ---- epilogue: warps 2..9; warp w reads TMEM lanes 32*(w%4) .. +31 (the lanes a warp may
  // touch), warps 2-5 the first half of the tile's columns, warps 6-9 the second half ----
  const int lane_group = warp & 3;
  constexpr int kColsPerWarp = BN / (EW / 4);
  const int col_begin = ((warp - 2) >> 2) * kColsPerWarp, col_end = col_begin + kColsPerWarp;
  // with split-K the raw accumulators go to the partial buffer (leading dimension m)
  const bool to_partial = p.splits > 1;
  const bool use_c = !to_partial && p.beta != 0.f;
  const float alpha = to_partial ? 1.0f : p.alpha;
  const long long ldc = to_partial ? (long long)p.m : p.ldc;
  int t = 0;
  for (int tile = work_first; tile < total_tiles; tile += work_stride, ++t) {
    THB_GEMM_TILE_COORDS(tile)
    const int acc = t % NACC;
    const int tile_m_own = PAIR ? 2 * tile_m + pair_rank : tile_m;   // this CTA's 128-row tile
    const int row = tile_m_own * THB_GEMM_BM + lane_group * 32 + lane;
    float* cb = (to_partial ? p.partial + (long long)split * p.partial_split_stride + (long long)batch * p.m * p.n
                            : p.c + (long long)batch * p.batch_stride_c) + row;
    const bool row_ok = row < p.m;
    // a tile that lies wholly inside C needs no per-element bounds checks
    const bool full = (tile_m_own + 1) * THB_GEMM_BM <= p.m && (tile_n + 1) * BN <= p.n;
    // Old values of C, 32 columns of this thread's row. They are read past L1 (ld.global.cg):
    // the 32 lines of one such block are ldc * 4 bytes apart and would fight for a few L1 sets.
    auto load_c = [&](float* dst, int col) {
      if (!use_c) return;
      const float* q = cb + (long long)col * ldc;
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; ++j) { dst[j] = __ldcg(q); q += ldc; }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) { dst[j] = (row_ok && col + j < p.n) ? __ldcg(q) : 0.f; q += ldc; }
      }
    };
    // C does not depend on the MMAs: with PREFETCH_C the first block of it is requested before
    // the wait, and each further block while the previous one is being combined and stored
    float cv[32], cn[32];
    if (PREFETCH_C) load_c(cv, tile_n * BN + col_begin);
    bool ok = thb_mbar_wait(thb_smem_u32(&bar_acc_full[acc]), (uint32_t)(t / NACC) & 1, abort_flag);
    if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, 3); }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
    for (int c0 = col_begin; c0 < col_end; c0 += 32) {
      uint32_t r[32];
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN + c0);
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
            "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
            "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
            "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
          : "r"(taddr));
      const int col0 = tile_n * BN + c0;
      if (PREFETCH_C) {
        if (c0 + 32 < col_end) load_c(cn, col0 + 32);
      } else {
        load_c(cv, col0);
      }
      // the accumulator registers are named as operands so that no use of them can be
      // scheduled before the wait
      asm volatile("tcgen05.wait::ld.sync.aligned;"
                   : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                     "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                     "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                     "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                   :
                   : "memory");
      float* q = cb + (long long)col0 * ldc;
      if (full) {
        if (use_c) {
#pragma unroll
          for (int j = 0; j < 32; ++j) { *q = alpha * __uint_as_float(r[j]) + p.beta * cv[j]; q += ldc; }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) { *q = alpha * __uint_as_float(r[j]); q += ldc; }
        }
      } else if (row_ok && col0 < p.n) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col0 + j < p.n) {
            float v = alpha * __uint_as_float(r[j]);
            if (use_c) v += p.beta * cv[j];
            *q = v;
          }
          q += ldc;
        }
      }
      if (PREFETCH_C) {
#pragma unroll
        for (int j = 0; j < 32; ++j) cv[j] = cn[j];
      }
    }
    // this warp is done reading the accumulator: hand it back to the MMA issuer
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      if (PAIR) thb_mbar_arrive_cluster_relaxed(thb_smem_u32(&bar_acc_empty[acc]), 0);
      else thb_mbar_arrive(thb_smem_u32(&bar_acc_empty[acc]));
    }
  }
}

// Persistent: CTA i works on tiles i, i + gridDim.x, ... The k loop of tile t+1
// overlaps the epilogue of tile t through two TMEM accumulators.
template <int BN, int BK, int STAGES, int EW, bool PREFETCH_C>
__global__ void __launch_bounds__(THB_GEMM_THREADS(EW), 1)
thb_gemm_3xtf32(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                ThbGemmParams p) {
  typedef ThbGemmCfg<BN, BK, STAGES> Cfg;
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment for the swizzle
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::kStage);
  uint64_t* bar_full = bars;                     // [STAGES] TMA -> MMA
  uint64_t* bar_empty = bars + STAGES;           // [STAGES] MMA -> TMA
  uint64_t* bar_acc_full = bars + 2 * STAGES;    // [2] MMA -> epilogue
  uint64_t* bar_acc_empty = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA (8 arrivals: one per warp)
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* never_set = abort_flag + 1;  // stays 0: for the waits of the exit path

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch * p.splits;  // work items
  const int group_sz = THB_GEMM_GROUP_M * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_full[s]), 1);
      thb_mbar_init(thb_smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      thb_mbar_init(thb_smem_u32(&bar_acc_full[a]), 1);
      thb_mbar_init(thb_smem_u32(&bar_acc_empty[a]), EW);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(thb_smem_u32(tmem_slot)),
                 "r"(Cfg::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer ----
      long long it = 0;  // k blocks issued so far, over all tiles of this CTA
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        THB_GEMM_TILE_COORDS(tile)
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t round = (uint32_t)(it / STAGES);
          if (it >= STAGES && !thb_mbar_wait(thb_smem_u32(&bar_empty[s]), (round - 1) & 1, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, 1); }
            ok = false;
            break;
          }
          const uint32_t full = thb_smem_u32(&bar_full[s]);
          uint8_t* st = smem + s * Cfg::kStage;
          thb_mbar_expect_tx(full, Cfg::kStage);
          const int k0 = kb * BK;
          thb_tma_load_3d(thb_smem_u32(st), &map_a, full, k0, tile_m * THB_GEMM_BM, batch * 2 + 0);
          thb_tma_load_3d(thb_smem_u32(st + Cfg::kTileA), &map_a, full, k0, tile_m * THB_GEMM_BM, batch * 2 + 1);
          thb_tma_load_3d(thb_smem_u32(st + 2 * Cfg::kTileA), &map_b, full, k0, tile_n * BN, batch * 2 + 0);
          thb_tma_load_3d(thb_smem_u32(st + 2 * Cfg::kTileA + Cfg::kTileB), &map_b, full, k0, tile_n * BN,
                          batch * 2 + 1);
        }
      }
      if (*abort_flag) {
        // do not leave while copies into this CTA's shared memory are in flight
        for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
          thb_mbar_wait(thb_smem_u32(&bar_full[j % STAGES]), (uint32_t)(j / STAGES) & 1, never_set);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      const uint32_t idesc = thb_umma_idesc_tf32(THB_GEMM_BM, BN);
      long long it = 0;
      int t = 0;  // tiles done by this CTA
      int fail_t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
        const int acc = t & 1;
        fail_t = t;
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        if (t >= 2 && !thb_mbar_wait(thb_smem_u32(&bar_acc_empty[acc]), ((uint32_t)(t >> 1) - 1) & 1, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, 4); }
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int split = tile % p.splits;
        const int kb_begin = split * p.kb_per_split;
        const int kb_end = min(p.kblocks, kb_begin + p.kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t round = (uint32_t)(it / STAGES);
          if (!thb_mbar_wait(thb_smem_u32(&bar_full[s]), round & 1, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, 2); }
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = thb_smem_u32(smem + s * Cfg::kStage);
          const uint64_t a_hi = thb_umma_desc<BK>(st);
          const uint64_t a_lo = thb_umma_desc<BK>(st + Cfg::kTileA);
          const uint64_t b_hi = thb_umma_desc<BK>(st + 2 * Cfg::kTileA);
          const uint64_t b_lo = thb_umma_desc<BK>(st + 2 * Cfg::kTileA + Cfg::kTileB);
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint64_t adv = (uint64_t)((kk * 32) >> 4);  // 8 tf32 = 32 bytes further along K
            thb_umma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, (kb != kb_begin) || (kk != 0));
            thb_umma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1);
            thb_umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1);
          }
          thb_umma_commit(thb_smem_u32(&bar_empty[s]));  // stage may be refilled
        }
        if (ok) thb_umma_commit(thb_smem_u32(&bar_acc_full[acc]));  // accumulator complete
      }
      if (!ok) {
        // after giving up: let the MMAs already issued drain before tensor memory is released
        thb_umma_commit(thb_smem_u32(&bar_acc_full[fail_t & 1]));
        thb_mbar_wait(thb_smem_u32(&bar_acc_full[fail_t & 1]), (uint32_t)(fail_t >> 1) & 1, never_set);
      }
    }
  } else {
    thb_gemm_epilogue_loop<BN, EW, PREFETCH_C>(p, tmem_base, bar_acc_full, bar_acc_empty, abort_flag);
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
  }
}

// Split-K fix-up: C = alpha * (P_0 + P_1 + ... in split order) + beta * C. C and the partials are
// column-major: a thread takes 4 consecutive rows (one 128-bit access; VEC = false: one row) of 4
// columns, all loads of which are issued before the first use. grid = (row groups, column groups, batch).
template <bool VEC>
static __global__ void __launch_bounds__(256)
thb_gemm_splitk_fixup(float* c, long long ldc, long long batch_stride_c, const float* partial,
                      long long partial_split_stride, int splits, int m, int n, float alpha, float beta) {
  constexpr int W = VEC ? 4 : 1;
  const int row = (blockIdx.x * 256 + threadIdx.x) * W;
  if (row >= m) return;
  const int col0 = blockIdx.y * 4;
  const float* part = partial + (long long)blockIdx.z * m * n + row;
  float* dst = c + (long long)blockIdx.z * batch_stride_c + row;
  float sum[4][W], old[4][W];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const bool ok = col0 + j < n;
    if (VEC) {
      const float4 v = ok ? __ldcg(reinterpret_cast<const float4*>(part + (long long)(col0 + j) * m)) : make_float4(0, 0, 0, 0);
      sum[j][0] = v.x; sum[j][1 % W] = v.y; sum[j][2 % W] = v.z; sum[j][3 % W] = v.w;
      const float4 o = (ok && beta != 0.f) ? *reinterpret_cast<const float4*>(dst + (long long)(col0 + j) * ldc) : make_float4(0, 0, 0, 0);
      old[j][0] = o.x; old[j][1 % W] = o.y; old[j][2 % W] = o.z; old[j][3 % W] = o.w;
    } else {
      sum[j][0] = ok ? __ldcg(part + (long long)(col0 + j) * m) : 0.f;
      old[j][0] = (ok && beta != 0.f) ? dst[(long long)(col0 + j) * ldc] : 0.f;
    }
  }
  for (int s = 1; s < splits; ++s) {
    float nxt[4][W];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool ok = col0 + j < n;
      const float* q = part + (long long)s * partial_split_stride + (long long)(col0 + j) * m;
      if (VEC) {
        const float4 v = ok ? __ldcg(reinterpret_cast<const float4*>(q)) : make_float4(0, 0, 0, 0);
        nxt[j][0] = v.x; nxt[j][1 % W] = v.y; nxt[j][2 % W] = v.z; nxt[j][3 % W] = v.w;
      } else {
        nxt[j][0] = ok ? __ldcg(q) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int w = 0; w < W; ++w) sum[j][w] += nxt[j][w];
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (col0 + j >= n) break;
    float v[W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
      v[w] = alpha * sum[j][w];
      if (beta != 0.f) v[w] += beta * old[j][w];
    }
    float* q = dst + (long long)(col0 + j) * ldc;
    if (VEC) *reinterpret_cast<float4*>(q) = make_float4(v[0], v[1 % W], v[2 % W], v[3 % W]);
    else *q = v[0];
  }
}
