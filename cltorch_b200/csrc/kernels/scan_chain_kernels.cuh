// Single-pass scan along the innermost dimension when there are too few rows for one warp per
// row to keep HBM busy (one long vector is the extreme case). The rows are cut into tiles of
// TILE elements; tile w (row-major over (row, piece)) is taken by CTA w mod G of a grid of G
// co-resident CTAs (cooperative launch, one per SM). Every tile is brought into shared memory
// twice: first for its total, then, a few tiles later and by then from L2, for the scan proper with
// the carry that the totals of the tiles before it give. HBM sees every element once in each
// direction: 8 bytes per element, against 12 for the three-phase form (totals, scan of totals,
// scan). While a tile waits for its carry it occupies L2, not shared memory, so the slack that
// absorbs the drift between CTAs costs no stage of the load pipeline.
//
// Same job as THClTensor_kernel_scanInnermostDim (reference src/lib/THClTensorMathScan.cl:52-139).
//
// The rows are seen as [row][n / 32][32 floats] through a tensor map with the 128-byte swizzle, so
// that a lane can own 16 consecutive elements (one inclusive scan over the lane totals per 512
// elements instead of one per 128) and still read and write shared memory without bank conflicts.
//
// Per CTA: warp 0 loads first visits into a ring of SA stages, warp 3 second visits into a ring of SB
// stages (cp.async.bulk.tensor, no multicast), warp 1 collects the carry of each tile, warp 2 returns
// scanned stages with cp.async.bulk.tensor stores, and two groups of warps do the arithmetic, each at
// its own pace:
//   pass A  (8 warps) the tile's total in double, published as one 8-byte word totals[w] (the word
//           itself says whether it has been written: the scratch is preset to all-ones, a pattern no
//           published total has); at most NSLOT tiles ahead of pass B;
//   pass B  (16 warps) carry + inclusive scan, written back into the stage.
// carry(w) = carry(w - G) (+) totals[w-G] (+) ... (+) totals[w-1], restricted to the tiles of w's own
// row: the additions are done in a fixed order (lane k folds entries k, k+32, ..., then a shuffle
// tree), so the result does not depend on which CTA was early. Totals never depend on carries,
// so no CTA waits for another's scan, only for its loads.
//
// A single vector whose length is not a multiple of 32 is scanned up to the last multiple; thb_scan_chain_tail
// continues over the remaining elements from the carry and the total of the last tile.
//
// Every wait is bounded (THB_GEMM_WAIT_LIMIT_NS). On expiry the waiter writes *status and sets
// the CTA's abort flag; waits in other CTAs notice *status and leave as well.
#pragma once
#include "gemm_kernels.cuh"  // mbarrier / TMA helpers
#include "scan_kernels.cuh"
#include "scan_strip_kernels.cuh"  // thb_tma_store_3d

#define THB_SCH_CWARPS 16
#define THB_SCH_AWARPS 8  // warps that add up tiles (1024 elements each); THB_SCH_CWARPS warps scan them (512 each)
#define THB_SCH_THREADS ((4 + THB_SCH_AWARPS + THB_SCH_CWARPS) * 32)
#define THB_SCH_MAX_CTAS 256  // the carry warp reads at most 8 totals per lane
#define THB_SCH_UNSET 0xFFFFFFFFFFFFFFFFull

// TMA copies with an L2 eviction priority: tiles on their first visit should stay in L2 until their second
// visit, which (like the results) has no later use.
__device__ __forceinline__ uint64_t thb_l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t thb_l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void thb_tma_load_3d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z,
                                                     uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void thb_tma_store_3d_hint(const CUtensorMap* map, uint32_t src, int x, int y, int z, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], [%1], %5;"
               ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z), "l"(policy)
               : "memory");
}
__device__ __forceinline__ unsigned long long thb_ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void thb_st_relaxed_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Status codes (family "strip scan"): 4 a carry never arrived, 5 load, 6 warp totals, 7 carry hand-over,
// 8 store, 9 a stage or carry slot never came free.
#define THB_SCH_SMEM_BYTES(TILE, SA, SB, NSLOT)                                                                   \
  (((SA) + (SB)) * (TILE) * 4 + 1024 /*alignment of the swizzled stages*/ +                                        \
   (NSLOT) * (THB_SCH_CWARPS + 1) * 8 /*warp offsets and carry per tile under way*/ +                              \
   (2 * (SA) + 3 * (SB) + 3 * (NSLOT)) * 8 /*barriers*/ + 16 /*flags*/)

template <class Op, int TILE, int SA, int SB, int NSLOT, int HINTS = 0>
__global__ void __launch_bounds__(THB_SCH_THREADS, 1)
thb_scan_chain(const __grid_constant__ CUtensorMap map_src, const __grid_constant__ CUtensorMap map_dst, thb_u32 n,
               thb_u32 nchunks, thb_i64 nwork, unsigned long long* totals, double* row_carry, int* status) {
  constexpr int STAGE_BYTES = TILE * 4;
  constexpr int WARP_ELEMS = TILE / THB_SCH_CWARPS;
  constexpr int LANE_ELEMS = WARP_ELEMS / 32;  // consecutive elements of a lane
  constexpr int PIECES = LANE_ELEMS / 4;       // float4 per lane and tile
  // NSLOT: how many tiles may be between their pass A and their pass B (the adding warps run ahead of the
  // scanning warps by at most that)
  static_assert(LANE_ELEMS == 16, "a scanning lane owns half a 128-byte row of the swizzled stage");
  static_assert(TILE == THB_SCH_AWARPS * 32 * 32, "an adding lane owns one 128-byte row of the stage");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* ring_a = smem;                     // tiles on their first visit: totals only
  uint8_t* ring_b = smem + SA * STAGE_BYTES;  // tiles on their second visit: scanned in place, then stored
  double* woff = (double*)(ring_b + SB * STAGE_BYTES);  // [slot][warp]
  double* carry_s = woff + NSLOT * THB_SCH_CWARPS;      // [slot]
  uint64_t* bar_full_a = (uint64_t*)(carry_s + NSLOT);
  uint64_t* bar_empty_a = bar_full_a + SA;
  uint64_t* bar_full_b = bar_empty_a + SA;
  uint64_t* bar_done_b = bar_full_b + SB;
  uint64_t* bar_empty_b = bar_done_b + SB;
  uint64_t* bar_tot = bar_empty_b + SB;   // [slot] every warp's total of the tile is in woff
  uint64_t* bar_pre = bar_tot + NSLOT;    // [slot] carry and warp offsets are in place
  uint64_t* bar_free = bar_pre + NSLOT;   // [slot] every warp has read them
  volatile int* abort_flag = (volatile int*)(bar_free + NSLOT);
  volatile int* never_set = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_full_a[s]), 1);
      thb_mbar_init(thb_smem_u32(&bar_empty_a[s]), THB_SCH_AWARPS);
    }
    for (int s = 0; s < SB; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_full_b[s]), 1);
      thb_mbar_init(thb_smem_u32(&bar_done_b[s]), THB_SCH_CWARPS);
      thb_mbar_init(thb_smem_u32(&bar_empty_b[s]), 1);
    }
    for (int s = 0; s < NSLOT; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_tot[s]), THB_SCH_AWARPS);
      thb_mbar_init(thb_smem_u32(&bar_pre[s]), 2);
      thb_mbar_init(thb_smem_u32(&bar_free[s]), THB_SCH_CWARPS);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const thb_i64 G = gridDim.x;
  const thb_i64 w_first = blockIdx.x;
  const int iters = w_first < nwork ? (int)((nwork - w_first + G - 1) / G) : 0;
  volatile int* gstatus = status;

#define THB_SCH_GIVE_UP(code)                                   \
  do {                                                          \
    if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, (code)); } \
  } while (0)

  if (warp == 0 || warp == 3) {
    // warp 0 brings every tile in for its first visit, warp 3 for its second (from L2 when all goes well:
    // the second visit follows the first by at most NSLOT tiles of every CTA).
    if (lane == 0) {
      const bool second = warp == 3;
      const int nst = second ? SB : SA;
      uint64_t* full_r = second ? bar_full_b : bar_full_a;
      uint64_t* empty_r = second ? bar_empty_b : bar_empty_a;
      uint8_t* ring = second ? ring_b : ring_a;
      const uint64_t policy = second ? thb_l2_policy_evict_first() : thb_l2_policy_evict_last();
      int i = 0;
      for (; i < iters; ++i) {
        const int s = i % nst;
        const uint32_t round = (uint32_t)(i / nst);
        if (i >= nst && !thb_mbar_wait(thb_smem_u32(&empty_r[s]), (round - 1) & 1, abort_flag)) {
          THB_SCH_GIVE_UP(9);
          break;
        }
        const thb_i64 w = w_first + (thb_i64)i * G;
        const thb_i64 row = w / nchunks;
        const thb_u32 c0 = (thb_u32)(w - row * nchunks) * TILE;
        const uint32_t full = thb_smem_u32(&full_r[s]);
        thb_mbar_expect_tx(full, STAGE_BYTES);  // 128-byte rows past the end of the row arrive as zeros
        if (HINTS & 1) thb_tma_load_3d_hint(thb_smem_u32(ring + s * STAGE_BYTES), &map_src, full, 0, (int)(c0 >> 5), (int)row, policy);
        else thb_tma_load_3d(thb_smem_u32(ring + s * STAGE_BYTES), &map_src, full, 0, (int)(c0 >> 5), (int)row);
      }
      if (*abort_flag) {
        // do not leave while copies into this CTA's shared memory are in flight
        for (int j = (i > nst ? i - nst : 0); j < i; ++j)
          thb_mbar_wait(thb_smem_u32(&full_r[j % nst]), (uint32_t)(j / nst) & 1, never_set);
      }
    }
  } else if (warp == 1) {
    // The totals of the next tile's predecessors are requested before this tile's are folded, so that
    // the trip to L2 is off the path from one carry to the next.
    constexpr int M = THB_SCH_MAX_CTAS / 32;
    double prev = Op::identity();
    unsigned long long nxt[M];
    thb_i64 w_n = w_first, row0_n = (w_n / nchunks) * nchunks, lo_n = (w_n - G > row0_n) ? w_n - G : row0_n;
    if (iters > 0) {
#pragma unroll
      for (int m = 0; m < M; ++m) nxt[m] = lo_n + lane + 32 * m < w_n ? thb_ld_relaxed_u64(totals + lo_n + lane + 32 * m) : 0ull;
    }
    for (int i = 0; i < iters; ++i) {
      const int slot = i % NSLOT;
      const uint32_t round = (uint32_t)(i / NSLOT);
      const thb_i64 w = w_n, row0 = row0_n, lo = lo_n;
      unsigned long long bits[M];
#pragma unroll
      for (int m = 0; m < M; ++m) bits[m] = nxt[m];
      if (i + 1 < iters) {
        w_n = w + G;
        row0_n = (w_n / nchunks) * nchunks;
        lo_n = (w_n - G > row0_n) ? w_n - G : row0_n;
#pragma unroll
        for (int m = 0; m < M; ++m) nxt[m] = lo_n + lane + 32 * m < w_n ? thb_ld_relaxed_u64(totals + lo_n + lane + 32 * m) : 0ull;
      }
      bool ok = true;
      bool missing = false;
#pragma unroll
      for (int m = 0; m < M; ++m) missing |= bits[m] == THB_SCH_UNSET;
      if (missing) {
        const unsigned long long t0 = thb_globaltimer_ns();
        for (uint32_t spin = 1; missing; ++spin) {
          missing = false;
#pragma unroll
          for (int m = 0; m < M; ++m) {
            if (bits[m] == THB_SCH_UNSET) {
              bits[m] = thb_ld_relaxed_u64(totals + lo + lane + 32 * m);
              missing |= bits[m] == THB_SCH_UNSET;
            }
          }
          if (missing && (spin & 31u) == 0 &&
              (*abort_flag || *gstatus != 0 || thb_globaltimer_ns() - t0 > THB_GEMM_WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
        }
      }
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) THB_SCH_GIVE_UP(4);
        break;
      }
      double acc = Op::identity();
#pragma unroll
      for (int m = 0; m < M; ++m)
        if (lo + lane + 32 * m < w) acc = Op::apply(acc, __longlong_as_double((long long)bits[m]));
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) acc = Op::apply(acc, __shfl_xor_sync(0xffffffffu, acc, off));
      prev = (w - G >= row0) ? Op::apply(prev, acc) : acc;
      // the slot is free once every warp has read the carry of the tile that used it before
      if (i >= NSLOT) ok = thb_mbar_wait(thb_smem_u32(&bar_free[slot]), (round - 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) THB_SCH_GIVE_UP(9);
        break;
      }
      if (lane == 0) {
        carry_s[slot] = prev;
        thb_mbar_arrive(thb_smem_u32(&bar_pre[slot]));
        if (row_carry && w - row0 == (thb_i64)nchunks - 1) row_carry[row0 / nchunks] = prev;  // what precedes the row's last tile
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      for (int i = 0; i < iters; ++i) {
        const int s = i % SB;
        const uint32_t round = (uint32_t)(i / SB);
        if (!thb_mbar_wait(thb_smem_u32(&bar_done_b[s]), round & 1, abort_flag)) {
          THB_SCH_GIVE_UP(8);
          break;
        }
        const thb_i64 w = w_first + (thb_i64)i * G;
        const thb_i64 row = w / nchunks;
        const thb_u32 c0 = (thb_u32)(w - row * nchunks) * TILE;
        // 128-byte rows past the end of the row are clipped by the TMA unit
        if (HINTS & 2) thb_tma_store_3d_hint(&map_dst, thb_smem_u32(ring_b + s * STAGE_BYTES), 0, (int)(c0 >> 5), (int)row, thb_l2_policy_evict_first());
        else thb_tma_store_3d(&map_dst, thb_smem_u32(ring_b + s * STAGE_BYTES), 0, (int)(c0 >> 5), (int)row);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        thb_mbar_arrive(thb_smem_u32(&bar_empty_b[s]));
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else if (warp < 4 + THB_SCH_AWARPS) {
    // pass A: the tile's total. A lane owns one 128-byte row of the stage (32 consecutive elements); the two
    // halves of the warp give the totals of two runs of 512 elements, the units of pass B.
    const int aw = warp - 4;
    const int srow = aw * 32 + lane;
    const thb_u32 e_lane = (thb_u32)srow * 32;
    for (int i = 0; i < iters; ++i) {
      const int s = i % SA;
      const int slot = i % NSLOT;
      bool ok = thb_mbar_wait(thb_smem_u32(&bar_full_a[s]), (uint32_t)(i / SA) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) THB_SCH_GIVE_UP(5);
        break;
      }
      const thb_i64 w = w_first + (thb_i64)i * G;
      const thb_u32 c0 = (thb_u32)(w % nchunks) * TILE;
      const thb_u32 len = min((thb_u32)TILE, n - c0);
      const uint8_t* tile = ring_a + s * STAGE_BYTES + srow * 128;
      double tot = Op::identity();
      if (e_lane < len) {  // n is a multiple of 32: a row of the stage is all inside or all outside
        double a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 t = *reinterpret_cast<const float4*>(tile + ((j ^ (srow & 7)) << 4));
          a[j] = Op::apply(Op::apply((double)t.x, (double)t.y), Op::apply((double)t.z, (double)t.w));
        }
        tot = Op::apply(Op::apply(Op::apply(a[0], a[1]), Op::apply(a[2], a[3])),
                        Op::apply(Op::apply(a[4], a[5]), Op::apply(a[6], a[7])));
      }
#pragma unroll
      for (int off = 1; off < 16; off <<= 1) tot = Op::apply(tot, __shfl_xor_sync(0xffffffffu, tot, off));
      // the slot is free once every scanning warp has read the offsets of the tile that used it before
      if (i >= NSLOT) ok = thb_mbar_wait(thb_smem_u32(&bar_free[slot]), (uint32_t)(i / NSLOT - 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) THB_SCH_GIVE_UP(9);
        break;
      }
      if ((lane & 15) == 0) woff[slot * THB_SCH_CWARPS + aw * 2 + (lane >> 4)] = tot;
      __syncwarp();
      if (lane == 0) {
        thb_mbar_arrive(thb_smem_u32(&bar_empty_a[s]));  // every lane's values are in: the stage can take the next tile
        thb_mbar_arrive(thb_smem_u32(&bar_tot[slot]));
      }
      if (aw == 0) {
        ok = thb_mbar_wait(thb_smem_u32(&bar_tot[slot]), (uint32_t)(i / NSLOT) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) THB_SCH_GIVE_UP(6);
          break;
        }
        if (lane == 0) {
          // the totals of the runs become what precedes each run inside the tile (read in pass B)
          double t = Op::identity();
#pragma unroll
          for (int k = 0; k < THB_SCH_CWARPS; ++k) {
            const double x = woff[slot * THB_SCH_CWARPS + k];
            woff[slot * THB_SCH_CWARPS + k] = t;
            t = Op::apply(t, x);
          }
          thb_mbar_arrive(thb_smem_u32(&bar_pre[slot]));
          unsigned long long bits = (unsigned long long)__double_as_longlong(t);
          if (bits == THB_SCH_UNSET) bits ^= 1ull;  // still a NaN; never the "not written" pattern
          thb_st_relaxed_u64(totals + w, bits);
        }
      }
    }
  } else {
    // pass B: carry + scan of the tile, in place.
    const int cw = warp - 4 - THB_SCH_AWARPS;
    // This lane's 16 consecutive elements: half of row `srow` of the stage ([TILE / 32] rows of 128 bytes whose
    // 16-byte pieces sit at (piece ^ (row & 7)): the 128-byte swizzle of the tensor map).
    const thb_u32 e_lane = cw * WARP_ELEMS + lane * LANE_ELEMS;
    const int srow = cw * (WARP_ELEMS / 32) + (lane >> 1);
    uint32_t piece_off[PIECES];
#pragma unroll
    for (int j = 0; j < PIECES; ++j) piece_off[j] = srow * 128 + ((((lane & 1) * 4 + j) ^ (srow & 7)) << 4);
    for (int j = 0; j < iters; ++j) {
      const int s = j % SB;
      const int slot = j % NSLOT;
      bool ok = thb_mbar_wait(thb_smem_u32(&bar_full_b[s]), (uint32_t)(j / SB) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) THB_SCH_GIVE_UP(5);
        break;
      }
      const thb_i64 w = w_first + (thb_i64)j * G;
      const thb_u32 c0 = (thb_u32)(w % nchunks) * TILE;
      const thb_u32 len = min((thb_u32)TILE, n - c0);
      uint8_t* tile = ring_b + s * STAGE_BYTES;
      const bool live = e_lane < len;
      // inclusive scans inside each float4, in double
      double q[PIECES][4];
      const float idf = (float)Op::identity();
#pragma unroll
      for (int u = 0; u < PIECES; ++u) {
        float4 t = make_float4(idf, idf, idf, idf);
        if (live) t = *reinterpret_cast<const float4*>(tile + piece_off[u]);
        q[u][0] = (double)t.x;
        q[u][1] = Op::apply(q[u][0], (double)t.y);
        q[u][2] = Op::apply(q[u][1], (double)t.z);
        q[u][3] = Op::apply(q[u][2], (double)t.w);
      }
      // what precedes each float4 inside the lane, and the lane's total
      double o[PIECES];
      o[0] = Op::identity();
#pragma unroll
      for (int u = 1; u < PIECES; ++u) o[u] = Op::apply(o[u - 1], q[u - 1][3]);
      double incl = Op::apply(o[PIECES - 1], q[PIECES - 1][3]);
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const double t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl = Op::apply(t, incl);
      }
      double excl = __shfl_up_sync(0xffffffffu, incl, 1);
      if (lane == 0) excl = Op::identity();
      // two arrivals: the carry (warp 1) and the offsets of the runs inside the tile (pass A)
      ok = thb_mbar_wait(thb_smem_u32(&bar_pre[slot]), (uint32_t)(j / NSLOT) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) THB_SCH_GIVE_UP(7);
        break;
      }
      const double run = Op::apply(carry_s[slot], woff[slot * THB_SCH_CWARPS + cw]);  // everything before this warp's elements
      __syncwarp();
      if (lane == 0) thb_mbar_arrive(thb_smem_u32(&bar_free[slot]));
      const double before = Op::apply(run, excl);
      if (live) {
#pragma unroll
        for (int u = 0; u < PIECES; ++u) {
          const double b = Op::apply(before, o[u]);
          *reinterpret_cast<float4*>(tile + piece_off[u]) =
              make_float4((float)Op::apply(b, q[u][0]), (float)Op::apply(b, q[u][1]), (float)Op::apply(b, q[u][2]),
                          (float)Op::apply(b, q[u][3]));
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // results visible to the TMA store
      __syncwarp();
      if (lane == 0) thb_mbar_arrive(thb_smem_u32(&bar_done_b[s]));
    }
  }
#undef THB_SCH_GIVE_UP
  __syncthreads();
}

// The up to 31 elements of a single vector that follow the part scanned by thb_scan_chain (n_main elements,
// nchunks tiles): running value = carry of the last tile (+) its total, then element by element.
template <class Op>
__global__ void thb_scan_chain_tail(float* dst, const float* src, thb_u32 n_main, thb_u32 n, thb_u32 nchunks,
                                    const unsigned long long* totals, const double* row_carry) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  double run = Op::apply(row_carry[0], __longlong_as_double((long long)totals[nchunks - 1]));
  for (thb_u32 k = n_main; k < n; ++k) {
    run = Op::apply(run, (double)src[k]);
    dst[k] = (float)run;
  }
}
