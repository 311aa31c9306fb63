// fp32 GEMM with the hi/lo split done inside the kernel: the operands cross HBM once.
//
// thb_gemm_3xtf32 (gemm_kernels.cuh) reads operands that a pre-pass has already split into
// hi = tf32(x) and lo = x - hi and laid out K-major. That pre-pass reads every operand once and
// writes it twice; for problems with little reuse (batched products with a short K, a few
// hundred rows against a large weight matrix) it costs as much as the product itself. Here
//
//  * TMA loads the RAW fp32 tiles straight from the caller's matrices, each operand in the
//    orientation it has in memory: K-major (unit stride along k: one box of BK x rows) or
//    MN-major (unit stride along the rows: one box of 32 rows x BK per 32 rows, in the 128-byte
//    swizzle with 32-byte atoms that the tensor core's MN-major descriptors expect for fp32). No transposition anywhere.
//  * two converter warps compute lo = x - (x with its 13 low mantissa bits cleared) for a landed
//    stage and write it to a second buffer at the same offset; the raw tile itself serves as hi
//    (the tensor core ignores those 13 bits). The conversion is position-preserving, so it is
//    independent of the swizzle pattern TMA applied.
//  * the MMA issuer then runs the same three tcgen05.mma.kind::tf32 per k step as
//    thb_gemm_3xtf32, with the A/B "major" bits of the instruction descriptor set per operand.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 epilogue (shared with
// thb_gemm_3xtf32), warps 10-11 converters. Barriers per stage: raw (TMA -> converters),
// conv (converters -> MMA), empty (MMA -> TMA). Every wait is bounded as in gemm_kernels.cuh;
// status codes 1-4 as there, 5 = a converter's wait for a landed stage, 6 = the MMA issuer's
// wait for a converted stage.
#pragma once

#include "gemm_kernels.cuh"

// Two converter warps: with TMA, the MMA issuer and eight epilogue warps that makes 384 threads, which
// leaves the epilogue the 168 registers per thread it needs to keep two 32-column blocks of C in
// flight (this kernel serves memory-bound problems, where the epilogue sets the pace).
#define THB_GEMM_CONV_WARPS 2
#define THB_GEMM_FUSED_THREADS (64 + 32 * 8 + 32 * THB_GEMM_CONV_WARPS)

template <int BN, int BK, int STAGES>
struct ThbGemmFusedCfg {
  static constexpr int kTileA = THB_GEMM_BM * BK * 4;
  static constexpr int kTileB = BN * BK * 4;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kStage = 2 * kTileA + 2 * kTileB;  // A raw (= hi), A lo, B raw (= hi), B lo
  static constexpr int kRawBytes = kTileA + kTileB;       // what TMA delivers per stage
  static constexpr int kSmem = STAGES * kStage + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

// Shared-memory descriptor of an MN-major tile of 32-bit elements: chunks of 32 rows (128 bytes)
// along M or N, each chunk BK k-rows of 128 bytes (so consecutive chunks are BK * 128 bytes apart:
// the leading byte offset). For 32-bit operands the tensor core transposes only from the 128-byte
// swizzle with 32-byte atoms (layout type 1: the 32-byte piece index of a row is XORed with the
// k-row index mod 4, TMA's CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B); that pattern repeats every 4
// k-rows, so groups of 4 k-rows are 512 bytes apart (the stride byte offset).
template <int BK>
__device__ __forceinline__ uint64_t thb_umma_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((BK * 128) >> 4) << 16;  // leading byte offset: next 32-row chunk
  d |= (uint64_t)(512 >> 4) << 32;         // stride byte offset: next group of 4 k-rows
  d |= (uint64_t)1 << 46;                  // descriptor version of sm_100
  d |= (uint64_t)1 << 61;                  // SWIZZLE_128B_BASE32B
  return d;
}

// hi = x rounded to TF32 (nearest, ties away from zero, as cvt.rna.tf32.f32 does for finite
// values: add half a TF32 unit to the magnitude and clear the 13 low bits), lo = x - hi.
__device__ __forceinline__ void thb_split_tf32(float x, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
  lo = x - hi;
}

// One converter thread's share of a tile of BYTES bytes: 16-byte chunks t, t + (converter threads), ...
// The tensor core reads a TF32 operand as the upper 19 bits of the fp32 word and ignores the 13 low
// mantissa bits. The raw tile therefore already IS a valid hi operand, hi = x with its low bits cut
// off, and only lo = x - hi has to be computed and written (exact in fp32; |lo| < 2^-10 |x|). That
// halves what the converters write to shared memory, which is what bounds this kernel. Against the
// rounded split of the other kernels the dropped terms are about twice as large (lo*lo ~ 2^-20,
// truncation of lo by the tensor core ~ 2^-21 relative): still two orders below the 1e-4 bar.
template <int BYTES>
__device__ __forceinline__ void thb_split_tile_lo(const uint8_t* raw, uint8_t* lo, int t) {
  constexpr int kPer = BYTES / 16 / (32 * THB_GEMM_CONV_WARPS);
  static_assert(kPer * 16 * 32 * THB_GEMM_CONV_WARPS == BYTES, "tile size must be a multiple of the converters' stride");
  float4 v[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) v[j] = *reinterpret_cast<const float4*>(raw + (t + j * 32 * THB_GEMM_CONV_WARPS) * 16);
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    float4 l;
    l.x = v[j].x - __uint_as_float(__float_as_uint(v[j].x) & 0xFFFFE000u);
    l.y = v[j].y - __uint_as_float(__float_as_uint(v[j].y) & 0xFFFFE000u);
    l.z = v[j].z - __uint_as_float(__float_as_uint(v[j].z) & 0xFFFFE000u);
    l.w = v[j].w - __uint_as_float(__float_as_uint(v[j].w) & 0xFFFFE000u);
    *reinterpret_cast<float4*>(lo + (t + j * 32 * THB_GEMM_CONV_WARPS) * 16) = l;
  }
}

// map_a / map_b describe the caller's matrices: K-major operand = (k, rows, batch) with box
// BK x rows-of-the-tile x 1; MN-major operand = (rows, k, batch) with box 32 x BK x 1.
template <int BN, int BK, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THB_GEMM_FUSED_THREADS, 1)
thb_gemm_3xtf32_fused(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      ThbGemmParams p) {
  typedef ThbGemmFusedCfg<BN, BK, STAGES> Cfg;
  constexpr int EW = 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::kStage);
  uint64_t* bar_raw = bars;                         // [STAGES] TMA -> converters
  uint64_t* bar_conv = bars + STAGES;               // [STAGES] converters -> MMA (one arrival per converter warp)
  uint64_t* bar_empty = bars + 2 * STAGES;          // [STAGES] MMA -> TMA
  uint64_t* bar_acc_full = bars + 3 * STAGES;       // [2] MMA -> epilogue
  uint64_t* bar_acc_empty = bars + 3 * STAGES + 2;  // [2] epilogue -> MMA
  uint32_t* tmem_slot = (uint32_t*)(bars + 3 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* never_set = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch * p.splits;
  const int group_sz = THB_GEMM_GROUP_M * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_raw[s]), 1);
      thb_mbar_init(thb_smem_u32(&bar_conv[s]), THB_GEMM_CONV_WARPS);
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
      // ---- TMA producer: raw fp32 tiles ----
      long long it = 0;
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
          const uint32_t full = thb_smem_u32(&bar_raw[s]);
          const uint32_t st = thb_smem_u32(smem + s * Cfg::kStage);
          thb_mbar_expect_tx(full, Cfg::kRawBytes);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < THB_GEMM_BM / 32; ++c)
              thb_tma_load_3d(st + c * (BK * 128), &map_a, full, tile_m * THB_GEMM_BM + c * 32, k0, batch);
          } else {
            thb_tma_load_3d(st, &map_a, full, k0, tile_m * THB_GEMM_BM, batch);
          }
          const uint32_t stb = st + 2 * Cfg::kTileA;
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              thb_tma_load_3d(stb + c * (BK * 128), &map_b, full, tile_n * BN + c * 32, k0, batch);
          } else {
            thb_tma_load_3d(stb, &map_b, full, k0, tile_n * BN, batch);
          }
        }
      }
      if (*abort_flag) {
        // do not leave while copies into this CTA's shared memory are in flight
        for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
          thb_mbar_wait(thb_smem_u32(&bar_raw[j % STAGES]), (uint32_t)(j / STAGES) & 1, never_set);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      const uint32_t idesc = thb_umma_idesc_tf32(THB_GEMM_BM, BN) | (A_MN ? (1u << 15) : 0u) | (B_MN ? (1u << 16) : 0u);
      long long it = 0;
      int t = 0;
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
          if (!thb_mbar_wait(thb_smem_u32(&bar_conv[s]), round & 1, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, 6); }
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = thb_smem_u32(smem + s * Cfg::kStage);
          const uint32_t stb = st + 2 * Cfg::kTileA;
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            // the kk-th group of 8 k values: 32 bytes further along a K-major row, 8 k-rows
            // (1024 bytes) further down an MN-major chunk
            const uint64_t a_hi = A_MN ? thb_umma_desc_mn<BK>(st + kk * 1024) : thb_umma_desc<BK>(st) + (uint64_t)((kk * 32) >> 4);
            const uint64_t a_lo = A_MN ? thb_umma_desc_mn<BK>(st + Cfg::kTileA + kk * 1024)
                                       : thb_umma_desc<BK>(st + Cfg::kTileA) + (uint64_t)((kk * 32) >> 4);
            const uint64_t b_hi = B_MN ? thb_umma_desc_mn<BK>(stb + kk * 1024) : thb_umma_desc<BK>(stb) + (uint64_t)((kk * 32) >> 4);
            const uint64_t b_lo = B_MN ? thb_umma_desc_mn<BK>(stb + Cfg::kTileB + kk * 1024)
                                       : thb_umma_desc<BK>(stb + Cfg::kTileB) + (uint64_t)((kk * 32) >> 4);
            thb_umma_tf32(d_tmem, a_lo, b_hi, idesc, (kb != kb_begin) || (kk != 0));
            thb_umma_tf32(d_tmem, a_hi, b_lo, idesc, 1);
            thb_umma_tf32(d_tmem, a_hi, b_hi, idesc, 1);
          }
          thb_umma_commit(thb_smem_u32(&bar_empty[s]));
        }
        if (ok) thb_umma_commit(thb_smem_u32(&bar_acc_full[acc]));
      }
      if (!ok) {
        thb_umma_commit(thb_smem_u32(&bar_acc_full[fail_t & 1]));
        thb_mbar_wait(thb_smem_u32(&bar_acc_full[fail_t & 1]), (uint32_t)(fail_t >> 1) & 1, never_set);
      }
    }
  } else if (warp < 2 + EW) {
    thb_gemm_epilogue_loop<BN, EW, true>(p, tmem_base, bar_acc_full, bar_acc_empty, abort_flag);
  } else {
    // ---- converters: lo beside the raw tile ----
    const int ct = threadIdx.x - 32 * (2 + EW);
    long long it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int split = tile % p.splits;
      const int kb_begin = split * p.kb_per_split;
      const int kb_end = min(p.kblocks, kb_begin + p.kb_per_split);
      for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
        const int s = (int)(it % STAGES);
        const uint32_t round = (uint32_t)(it / STAGES);
        bool got = thb_mbar_wait(thb_smem_u32(&bar_raw[s]), round & 1, abort_flag);
        if (!got && !*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, 5); }
        got = __all_sync(0xffffffffu, got);
        if (!got) { ok = false; break; }
        uint8_t* st = smem + s * Cfg::kStage;
        thb_split_tile_lo<Cfg::kTileA>(st, st + Cfg::kTileA, ct);
        thb_split_tile_lo<Cfg::kTileB>(st + 2 * Cfg::kTileA, st + 2 * Cfg::kTileA + Cfg::kTileB, ct);
        // the tensor core reads shared memory through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) thb_mbar_arrive(thb_smem_u32(&bar_conv[s]));
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
  }
}
