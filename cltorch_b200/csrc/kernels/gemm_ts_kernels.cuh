// fp32 GEMM for long-K problems with the A' operand fed to the tensor core from TENSOR MEMORY.
//
// The pre-pass of thb_gemm_3xtf32 reads every operand once and writes it twice before the product
// starts; for "few rows x large weight matrix" that costs a quarter of the call. Here the large
// operand is never pre-processed:
//
//  * A' (the operand whose rows run along C's unit stride) is loaded RAW by TMA in the orientation it
//    has in memory (MN-major: a box of 128 rows x BK, no swizzle; K-major: BK x 128 rows with the
//    64-byte swizzle), and four converter warps - one per quarter of
//    the 128 TMEM lanes - read it (thread = row, conflict-free), split it into hi = tf32(x) and
//    lo = x - hi in registers and store both with tcgen05.st into a ring of TMEM slots
//    (2 x BK columns per stage). It never goes back to shared memory and is not pre-processed in HBM.
//  * B' comes pre-split (hi, lo; K-major; 64-byte swizzle) from the small pre-pass, as in
//    thb_gemm_3xtf32, and is the only operand the MMAs read from shared memory (24 KB per k step
//    instead of 36 KB). Measured: the tensor pipe is ~90-92 % busy, the same as with both operands
//    in shared memory, so those reads were not what keeps it from 100 %.
//  * the MMA issuer runs  a_lo*b_hi + a_hi*b_lo + a_hi*b_hi  per k step with A addressed in TMEM.
//
// One 128 x BN accumulator (TMEM: BN columns + STAGES slots of 2*BK columns <= 512): the
// epilogue of a tile does not overlap the next tile's main loop, which costs about 1 % when a
// tile's k loop is hundreds of microseconds long; the host uses this kernel only for long K.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 epilogue (shared code), warps 10-13
// converters (warp w serves TMEM lanes 32*(w%4) .. +31). Barriers per stage: raw (TMA ->
// converters), conv (converters -> MMA), empty (MMA -> TMA; frees the shared-memory stage and the
// TMEM slot together). Bounded waits and status codes as in gemm_fused_kernels.cuh.
#pragma once

#include "gemm_fused_kernels.cuh"

#define THB_GEMM_TS_CONV_WARPS 4   // one per quarter of the TMEM lanes
#define THB_GEMM_TS_THREADS (64 + 32 * 8 + 32 * THB_GEMM_TS_CONV_WARPS)

template <int BN, int BK, int STAGES>
struct ThbGemmTsCfg {
  static constexpr int kTileA = THB_GEMM_BM * BK * 4;   // raw A', [BK][128] floats
  static constexpr int kTileB = BN * BK * 4;            // one of B'_hi, B'_lo
  static constexpr int kStage = kTileA + 2 * kTileB;
  static constexpr int kAccCols = BN;                   // one accumulator
  static constexpr int kSlotCols = 2 * BK;              // hi then lo of one k block
  static constexpr int kTmemCols = 512;
  static_assert(kAccCols + STAGES * kSlotCols <= kTmemCols, "tensor memory budget");
  static constexpr int kSmem = STAGES * kStage + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

// A in tensor memory, B through a shared-memory descriptor.
__device__ __forceinline__ void thb_umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16 consecutive columns of this thread's TMEM lane.
__device__ __forceinline__ void thb_tmem_store16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// map_a: the caller's A'. A_KMAJOR = false (unit stride along the rows): (rows, k, batch), box 128 x BK x 1,
//        no swizzle; a converter thread reads its row's k-th element from k-row k (a warp reads 128
//        consecutive bytes). A_KMAJOR = true (unit stride along k): (k, rows, batch), box BK x 128 x 1
//        with the 64-byte swizzle; a thread reads the four 16-byte pieces of its own 64-byte row, whose
//        positions the swizzle spreads over all banks (piece j of row r sits at j ^ ((r >> 1) & 3)).
// map_b: the pre-split B' as in thb_gemm_3xtf32 ([2 * batch][n][Kp], box BK x BN x 1, 64-byte swizzle).
template <int BN, int BK, int STAGES, bool A_KMAJOR>
__global__ void __launch_bounds__(THB_GEMM_TS_THREADS, 1)
thb_gemm_3xtf32_ts(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, ThbGemmParams p) {
  typedef ThbGemmTsCfg<BN, BK, STAGES> Cfg;
  static_assert(BK == 16, "one tcgen05.st of 16 columns per half");
  constexpr int EW = 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::kStage);
  uint64_t* bar_raw = bars;                         // [STAGES] TMA -> converters
  uint64_t* bar_conv = bars + STAGES;               // [STAGES] converters -> MMA
  uint64_t* bar_empty = bars + 2 * STAGES;          // [STAGES] MMA -> TMA
  uint64_t* bar_acc_full = bars + 3 * STAGES;       // [2] (only [0] used) MMA -> epilogue
  uint64_t* bar_acc_empty = bars + 3 * STAGES + 2;  // [2] (only [0] used) epilogue -> MMA
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
      thb_mbar_init(thb_smem_u32(&bar_conv[s]), THB_GEMM_TS_CONV_WARPS);
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
  const uint32_t tmem_a = tmem_base + (uint32_t)Cfg::kAccCols;  // first column of the A' slots

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: raw A', pre-split B' ----
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
          thb_mbar_expect_tx(full, Cfg::kStage);
          const int k0 = kb * BK;
          if (A_KMAJOR) thb_tma_load_3d(st, &map_a, full, k0, tile_m * THB_GEMM_BM, batch);
          else thb_tma_load_3d(st, &map_a, full, tile_m * THB_GEMM_BM, k0, batch);
          thb_tma_load_3d(st + Cfg::kTileA, &map_b, full, k0, tile_n * BN, batch * 2 + 0);
          thb_tma_load_3d(st + Cfg::kTileA + Cfg::kTileB, &map_b, full, k0, tile_n * BN, batch * 2 + 1);
        }
      }
      if (*abort_flag) {
        for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
          thb_mbar_wait(thb_smem_u32(&bar_raw[j % STAGES]), (uint32_t)(j / STAGES) & 1, never_set);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      const uint32_t idesc = thb_umma_idesc_tf32(THB_GEMM_BM, BN);
      long long it = 0;
      int t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
        // the one accumulator is free again when the epilogue of the previous tile has read it
        if (t >= 1 && !thb_mbar_wait(thb_smem_u32(&bar_acc_empty[0]), ((uint32_t)t - 1) & 1, abort_flag)) {
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
          const uint32_t stb = thb_smem_u32(smem + s * Cfg::kStage) + Cfg::kTileA;
          const uint64_t b_hi = thb_umma_desc<BK>(stb);
          const uint64_t b_lo = thb_umma_desc<BK>(stb + Cfg::kTileB);
          const uint32_t a_hi = tmem_a + (uint32_t)(s * Cfg::kSlotCols), a_lo = a_hi + BK;
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint64_t adv = (uint64_t)((kk * 32) >> 4);  // 8 tf32 = 32 bytes further along K
            thb_umma_tf32_ts(tmem_base, a_lo + kk * 8, b_hi + adv, idesc, (kb != kb_begin) || (kk != 0));
            thb_umma_tf32_ts(tmem_base, a_hi + kk * 8, b_lo + adv, idesc, 1);
            thb_umma_tf32_ts(tmem_base, a_hi + kk * 8, b_hi + adv, idesc, 1);
          }
          thb_umma_commit(thb_smem_u32(&bar_empty[s]));
        }
        if (ok) thb_umma_commit(thb_smem_u32(&bar_acc_full[0]));
      }
      if (!ok) {
        // let the MMAs already issued drain before tensor memory is released: bar_acc_full[0] has
        // completed t phases so far, the commit below completes one more
        thb_umma_commit(thb_smem_u32(&bar_acc_full[0]));
        thb_mbar_wait(thb_smem_u32(&bar_acc_full[0]), (uint32_t)t & 1, never_set);
      }
    }
  } else if (warp < 2 + EW) {
    thb_gemm_epilogue_loop<BN, EW, true, 1>(p, tmem_base, bar_acc_full, bar_acc_empty, abort_flag);
  } else {
    // ---- converters: raw A' (shared memory) -> hi, lo (tensor memory) ----
    const int q = warp & 3;                 // the quarter of the TMEM lanes this warp may touch
    const int row = q * 32 + lane;          // row of the tile = TMEM lane
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
        uint32_t hi[BK], lo[BK];
        if (A_KMAJOR) {
          const uint8_t* raw = smem + s * Cfg::kStage + row * (BK * 4);  // [128][BK], 16-byte pieces swizzled
#pragma unroll
          for (int j = 0; j < BK / 4; ++j) {
            const float4 x = *reinterpret_cast<const float4*>(raw + ((j ^ ((row >> 1) & 3)) << 4));
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float h, l;
              thb_split_tf32(xs[e], h, l);
              hi[4 * j + e] = __float_as_uint(h);
              lo[4 * j + e] = __float_as_uint(l);
            }
          }
        } else {
          const float* raw = reinterpret_cast<const float*>(smem + s * Cfg::kStage) + row;  // [k][128]
#pragma unroll
          for (int k = 0; k < BK; ++k) {
            float h, l;
            thb_split_tf32(raw[k * THB_GEMM_BM], h, l);
            hi[k] = __float_as_uint(h);
            lo[k] = __float_as_uint(l);
          }
        }
        // the MMAs that read this slot one round ago have completed: the producer waited for their
        // commit before it refilled the stage whose arrival was just observed
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem_a + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * Cfg::kSlotCols);
        thb_tmem_store16(taddr, hi);
        thb_tmem_store16(taddr + BK, lo);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
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
