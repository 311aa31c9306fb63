// The shared-memory-split GEMM of gemm_fused_kernels.cuh on PAIRS of CTAs (thread-block clusters of
// two, tcgen05 cta_group::2): one 256 x 256 output tile per pair.
//
// Why: the single-CTA kernel is bound by the SM's shared-memory data path on short-K problems - per
// 16-deep stage 24 KB from TMA, 48 KB through the converter warps and 72 KB of operand reads by six
// MMAs (each reads its 128 x 8 slice of A and the whole 256 x 8 slice of B). In a pair each CTA holds
// its own 128 rows of A' and only HALF of the B' tile (128 of the 256 rows); a cta_group::2 MMA feeds
// both tensor cores from both halves, so per CTA and stage: 16 KB from TMA, 32 KB converted, 48 KB of
// operand reads - a third less, and a stage is 32 KB instead of 48 KB (six stages in flight).
//
// Roles per CTA as in the single-CTA kernel (warp 0 TMA producer for its own tiles, warps 2-9
// epilogue for its own 128 rows, warps 10-11 converters for its own stage); the MMAs of a pair are
// issued by one thread of the cluster's first CTA. Barriers sit at the same shared-memory offsets
// in both CTAs:
//   raw[s]    local   TMA -> converters of the same CTA
//   conv[s]   leader  one arrival per converter warp of BOTH CTAs (the second CTA arrives remotely)
//   empty[s]  both    the leader commits the stage's MMAs to its own and to the peer's barrier
//   acc_full  both    same, once per tile
//   acc_empty leader  one arrival per epilogue warp of BOTH CTAs
// No multicast anywhere: the peer's barriers are addressed explicitly (mapa), every CTA loads
// its own tiles. All waits are bounded; both CTAs always reach the cluster barriers at entry and
// exit, so a CTA that gave up does not strand its partner. Status codes as in
// gemm_fused_kernels.cuh.
#pragma once

#include "gemm_fused_kernels.cuh"

template <int BK, int STAGES>
struct ThbGemmPairCfg {
  static constexpr int kBN = 256;                             // of the pair; each CTA holds 128 rows of B'
  static constexpr int kTileA = THB_GEMM_BM * BK * 4;
  static constexpr int kTileB = (kBN / 2) * BK * 4;           // this CTA's half
  static constexpr int kTmemCols = 2 * kBN;
  static constexpr int kStage = 2 * kTileA + 2 * kTileB;      // A raw (= hi), A lo, B-half raw, B-half lo
  static constexpr int kRawBytes = kTileA + kTileB;
  static constexpr int kSmem = STAGES * kStage + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

__device__ __forceinline__ void thb_umma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Makes the barrier at offset `bar` in BOTH CTAs of the pair complete a phase when the MMAs issued so far
// have finished: one commit per barrier (the peer's is addressed through mapa).
__device__ __forceinline__ void thb_umma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b32 peer;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "mapa.shared::cluster.u32 peer, %0, 1;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [peer];\n\t}"
      ::"r"(bar)
      : "memory");
}

// map_a: the caller's A' (as for the single-CTA kernel: K-major box BK x 128, or MN-major box 32 x BK).
// map_b: the caller's B' with a box of 128 rows (K-major) or 32 rows (MN-major).
// p.tiles_m counts 256-row tile pairs here.
template <int BK, int STAGES, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THB_GEMM_FUSED_THREADS, 1)
thb_gemm_3xtf32_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, ThbGemmParams p) {
  typedef ThbGemmPairCfg<BK, STAGES> Cfg;
  constexpr int BN = Cfg::kBN;
  constexpr int EW = 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::kStage);
  uint64_t* bar_raw = bars;
  uint64_t* bar_conv = bars + STAGES;
  uint64_t* bar_empty = bars + 2 * STAGES;
  uint64_t* bar_acc_full = bars + 3 * STAGES;
  uint64_t* bar_acc_empty = bars + 3 * STAGES + 2;
  uint32_t* tmem_slot = (uint32_t*)(bars + 3 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* never_set = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)(blockIdx.x & 1);            // position in the pair (cluster dims 2 x 1 x 1)
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch * p.splits;
  const int group_sz = THB_GEMM_GROUP_M * p.tiles_n;
  const int work_first = (int)(blockIdx.x >> 1), work_stride = (int)(gridDim.x >> 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_raw[s]), 1);
      thb_mbar_init(thb_smem_u32(&bar_conv[s]), 2 * THB_GEMM_CONV_WARPS);
      thb_mbar_init(thb_smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      thb_mbar_init(thb_smem_u32(&bar_acc_full[a]), 1);
      thb_mbar_init(thb_smem_u32(&bar_acc_empty[a]), 2 * EW);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(thb_smem_u32(tmem_slot)),
                 "r"(Cfg::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  thb_cluster_sync();  // the partner's barriers exist before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: this CTA's 128 rows of A' and its 128 of the 256 rows of B' ----
      long long it = 0;
      bool ok = true;
      for (int tile = work_first; tile < total_tiles && ok; tile += work_stride) {
        THB_GEMM_TILE_COORDS(tile)
        const int row_a = (2 * tile_m + rank) * THB_GEMM_BM, row_b = tile_n * BN + rank * (BN / 2);
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
            for (int c = 0; c < THB_GEMM_BM / 32; ++c) thb_tma_load_3d(st + c * (BK * 128), &map_a, full, row_a + c * 32, k0, batch);
          } else {
            thb_tma_load_3d(st, &map_a, full, k0, row_a, batch);
          }
          const uint32_t stb = st + 2 * Cfg::kTileA;
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 2 / 32; ++c) thb_tma_load_3d(stb + c * (BK * 128), &map_b, full, row_b + c * 32, k0, batch);
          } else {
            thb_tma_load_3d(stb, &map_b, full, k0, row_b, batch);
          }
        }
      }
      if (*abort_flag) {
        for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
          thb_mbar_wait(thb_smem_u32(&bar_raw[j % STAGES]), (uint32_t)(j / STAGES) & 1, never_set);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- MMA issuer of the pair ----
      const uint32_t idesc = thb_umma_idesc_tf32(2 * THB_GEMM_BM, BN) | (A_MN ? (1u << 15) : 0u) | (B_MN ? (1u << 16) : 0u);
      long long it = 0;
      int t = 0;
      int fail_t = 0;
      bool ok = true;
      for (int tile = work_first; tile < total_tiles && ok; tile += work_stride, ++t) {
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
            const uint64_t a_hi = A_MN ? thb_umma_desc_mn<BK>(st + kk * 1024) : thb_umma_desc<BK>(st) + (uint64_t)((kk * 32) >> 4);
            const uint64_t a_lo = A_MN ? thb_umma_desc_mn<BK>(st + Cfg::kTileA + kk * 1024)
                                       : thb_umma_desc<BK>(st + Cfg::kTileA) + (uint64_t)((kk * 32) >> 4);
            const uint64_t b_hi = B_MN ? thb_umma_desc_mn<BK>(stb + kk * 1024) : thb_umma_desc<BK>(stb) + (uint64_t)((kk * 32) >> 4);
            const uint64_t b_lo = B_MN ? thb_umma_desc_mn<BK>(stb + Cfg::kTileB + kk * 1024)
                                       : thb_umma_desc<BK>(stb + Cfg::kTileB) + (uint64_t)((kk * 32) >> 4);
            thb_umma_tf32_pair(d_tmem, a_lo, b_hi, idesc, (kb != kb_begin) || (kk != 0));
            thb_umma_tf32_pair(d_tmem, a_hi, b_lo, idesc, 1);
            thb_umma_tf32_pair(d_tmem, a_hi, b_hi, idesc, 1);
          }
          thb_umma_commit_pair(thb_smem_u32(&bar_empty[s]));
        }
        if (ok) thb_umma_commit_pair(thb_smem_u32(&bar_acc_full[acc]));
      }
      if (!ok) {
        thb_umma_commit_pair(thb_smem_u32(&bar_acc_full[fail_t & 1]));
        thb_mbar_wait(thb_smem_u32(&bar_acc_full[fail_t & 1]), (uint32_t)(fail_t >> 1) & 1, never_set);
      }
    }
  } else if (warp < 2 + EW) {
    thb_gemm_epilogue_loop<BN, EW, true, 2, true>(p, tmem_base, bar_acc_full, bar_acc_empty, abort_flag);
  } else {
    // ---- converters: lo beside this CTA's raw tiles; done -> the leader's barrier ----
    const int ct = threadIdx.x - 32 * (2 + EW);
    long long it = 0;
    bool ok = true;
    for (int tile = work_first; tile < total_tiles && ok; tile += work_stride) {
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
        // fence.proxy.async makes this thread's shared-memory writes visible to the tensor core of this
        // SM; the arrival itself then needs no cluster-scope release (measured: with one, the converters
        // spent longer in the fence than in the conversion).
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) thb_mbar_arrive(thb_smem_u32(&bar_conv[s]));
          else thb_mbar_arrive_cluster_relaxed(thb_smem_u32(&bar_conv[s]), 0);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  thb_cluster_sync();  // neither CTA releases tensor memory or leaves while its partner may still use it
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
  }
}
