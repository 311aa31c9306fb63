// Pointwise apply when every operand is the same R x C matrix and at least one of them is
// column-major-like (a transpose view), for matrices large enough to keep every SM busy.
//
// Same job as thb_apply_tile2d_v4, i.e. what the reference does with one work-item per element and
// a div/mod chain per operand (src/lib/THClApply.cl:47-102), but no thread touches global memory:
// a persistent CTA per SM walks 64 x 64 tiles; warp 0 asks the TMA unit for the tile of each input
// (four 32 x 32 boxes per operand, 128-byte swizzle, each in the operand's own orientation), eight
// consumer warps (two groups on alternate tiles) combine the staged tiles in shared memory, and warp 9 hands the result tile back
// to the TMA unit, which writes it in the output's orientation. The transposition happens in how a
// thread addresses shared memory: thread = one row r of a box; a row-major box is read as 16-byte
// chunks (r, 4ch..4ch+3), a column-major box as four scalars (4ch+j, r). With the swizzle both are
// free of bank conflicts.
//
// Stage s of the ring holds NT operand slots of 16 KB; slot 0 is the output tile (loaded first only
// if the operator reads it). Barriers: full[s] (loads landed), done[s] (the consumer warps of the tile
// wrote their results), empty[s] (the store has read the stage). Every wait is bounded; on expiry the
// waiter records a code in *status, raises the CTA's abort flag and all roles leave after the
// copies in flight have landed.
//
// Like apply_kernels.cuh this text is also compiled by NVRTC for user expressions: the #include
// lines are skipped there (the pieces are concatenated instead).
#pragma once
#ifndef __CUDACC_RTC__
#include "tma_pipeline.cuh"
#include "apply_kernels.cuh"
#endif

#define THB_AT_TILE 64
#define THB_AT_BOX 32
#define THB_AT_BOX_BYTES (THB_AT_BOX * THB_AT_BOX * 4)
#define THB_AT_OPERAND_BYTES (4 * THB_AT_BOX_BYTES)
#define THB_AT_STAGES(NT) (12 / (NT))  // 192 KB of stages whatever the operand count
#define THB_AT_THREADS 320
#ifndef THB_AT_GROUPS
#define THB_AT_GROUPS 2  // consumer groups: each takes every THB_AT_GROUPS-th tile of the CTA
#endif
#define THB_AT_SMEM(NT) (THB_AT_STAGES(NT) * (NT) * THB_AT_OPERAND_BYTES + 1024 /*alignment*/ + 512 /*barriers*/)

struct ThbTileTma {
  thb_u32 R, C;
  thb_u32 tilesC;  // ceil(C / 64)
  thb_u32 ntiles;  // ceil(R / 64) * tilesC
  int colmajor;    // bit q: operand q is column-major-like (its tensor map has R innermost)
  thb_u32 tilesR;  // ceil(R / 64)
  thb_u32 band;    // tiles are visited in bands of this many tile rows, down the rows first (<= 1: row by row)
  int* status;
};

// Tile t in visiting order -> its first row and column. The CTAs of one round hold consecutive t:
// with bands they cover a patch of `band` x (CTAs / band) tiles, so that the requests in flight at
// one time fall into long runs of the row-major AND of the column-major operands.
__device__ __forceinline__ void thb_at_tile_origin(const ThbTileTma& P, thb_u32 t, int* r0, int* c0) {
  thb_u32 tr = t / P.tilesC, tc = t - tr * P.tilesC;
  if (P.band > 1) {
    const thb_u32 per_band = P.band * P.tilesC;
    const thb_u32 b = t / per_band, in_band = t - b * per_band;
    const thb_u32 rows_here = min(P.band, P.tilesR - b * P.band);
    tc = in_band / rows_here;
    tr = b * P.band + (in_band - tc * rows_here);
  }
  *r0 = (int)(tr * THB_AT_TILE);
  *c0 = (int)(tc * THB_AT_TILE);
}

template <class Op, int NT>
__global__ void __launch_bounds__(THB_AT_THREADS, 1)
thb_apply_tile_tma(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                   const __grid_constant__ CUtensorMap map2, ThbTileTma P, ThbScalars s) {
  thb_grid_dependency_sync();
  constexpr int kStage = NT * THB_AT_OPERAND_BYTES;
  constexpr int kStages = THB_AT_STAGES(NT);
  constexpr int kFirstLoaded = Op::kReadsOut ? 0 : 1;
  constexpr int kLoaded = NT - kFirstLoaded;  // the host only picks this kernel when kLoaded >= 1
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bar_full = (uint64_t*)(smem + kStages * kStage);
  uint64_t* bar_empty = bar_full + kStages;
  uint64_t* bar_done = bar_empty + kStages;
  volatile int* abort_flag = (volatile int*)(bar_done + kStages);
  volatile int* never_set = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      thb_mbar_init(thb_smem_u32(&bar_full[i]), 1);
      thb_mbar_init(thb_smem_u32(&bar_empty[i]), 1);
      thb_mbar_init(thb_smem_u32(&bar_done[i]), 8 / THB_AT_GROUPS);  // one arrival per consumer warp of a group
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 0) {
    // ---- loads ----
    if (lane == 0) {
      long long it = 0;
      for (thb_u32 t = blockIdx.x; t < P.ntiles; t += gridDim.x, ++it) {
        const int st = (int)(it % kStages);
        const uint32_t round = (uint32_t)(it / kStages);
        if (it >= kStages && !thb_mbar_wait(thb_smem_u32(&bar_empty[st]), (round - 1) & 1, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; if (P.status) atomicCAS(P.status, 0, 11); }
          break;
        }
        int r0, c0;
        thb_at_tile_origin(P, t, &r0, &c0);
        const uint32_t full = thb_smem_u32(&bar_full[st]);
        thb_mbar_expect_tx(full, kLoaded * THB_AT_OPERAND_BYTES);  // parts of a box past the edges arrive as zeros
#pragma unroll
        for (int q = kFirstLoaded; q < NT; ++q) {
          const CUtensorMap* map = q == 0 ? &map0 : (q == 1 ? &map1 : &map2);
          const bool col = (P.colmajor >> q) & 1;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int r = r0 + THB_AT_BOX * (b >> 1), c = c0 + THB_AT_BOX * (b & 1);
            const uint32_t dst = thb_smem_u32(smem + st * kStage + q * THB_AT_OPERAND_BYTES + b * THB_AT_BOX_BYTES);
            thb_tma_load_2d(dst, map, full, col ? r : c, col ? c : r);
          }
        }
      }
      if (*abort_flag) {
        // do not leave while copies into this CTA's shared memory are in flight
        for (long long j = (it > kStages ? it - kStages : 0); j < it; ++j)
          thb_mbar_wait(thb_smem_u32(&bar_full[j % kStages]), (uint32_t)(j / kStages) & 1, never_set);
      }
    }
  } else if (warp == 9) {
    // ---- stores ----
    if (lane == 0) {
      long long it = 0;
      for (thb_u32 t = blockIdx.x; t < P.ntiles; t += gridDim.x, ++it) {
        const int st = (int)(it % kStages);
        const uint32_t round = (uint32_t)(it / kStages);
        if (!thb_mbar_wait(thb_smem_u32(&bar_done[st]), round & 1, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; if (P.status) atomicCAS(P.status, 0, 13); }
          break;
        }
        int r0, c0;
        thb_at_tile_origin(P, t, &r0, &c0);
        const bool col = P.colmajor & 1;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int r = r0 + THB_AT_BOX * (b >> 1), c = c0 + THB_AT_BOX * (b & 1);
          if ((thb_u32)r < P.R && (thb_u32)c < P.C)  // a store never starts outside the matrix; the unit clips the rest
            thb_tma_store_2d(&map0, thb_smem_u32(smem + st * kStage + b * THB_AT_BOX_BYTES), col ? r : c, col ? c : r);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // once the store has read the stage it may be refilled (this thread has nothing else to do meanwhile)
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        thb_mbar_arrive(thb_smem_u32(&bar_empty[st]));
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else {
    // ---- consumers: THB_AT_GROUPS groups of warps work on different tiles at the same time, so that
    // one group's barrier and fence latencies hide behind the other's work. Within a group a box
    // belongs to one warp (or a pair); lane = row of the box, a thread takes 4-column chunks. ----
    float p1 = 0.f, p2 = 0.f;
    if (s.pointTensor1) p1 = *s.pointTensor1;
    if (s.pointTensor2) p2 = *s.pointTensor2;
    constexpr int kWarpsPerBox = 8 / THB_AT_GROUPS / 4;  // 2 or 1
    constexpr int kChunks = 8 / kWarpsPerBox;            // chunks of a box per thread
    const int cw = warp - 1;
    const int group = cw / (8 / THB_AT_GROUPS), gw = cw % (8 / THB_AT_GROUPS);
    const int box = gw / kWarpsPerBox, half = gw % kWarpsPerBox;
    // byte offsets inside a box: row-major chunk (lane, ch) and column-major element (4ch+j, lane)
    const uint32_t row_base = (uint32_t)lane * 128u;
    const uint32_t row_xor = (uint32_t)(lane & 7);
    const uint32_t col_chunk = (uint32_t)(lane >> 2), col_in = (uint32_t)(lane & 3) * 4u;
    long long it = group;
    for (unsigned long long t = blockIdx.x + (unsigned long long)group * gridDim.x; t < P.ntiles;
         t += (unsigned long long)THB_AT_GROUPS * gridDim.x, it += THB_AT_GROUPS) {
      const int st = (int)(it % kStages);
      const uint32_t round = (uint32_t)(it / kStages);
      bool got = thb_mbar_wait(thb_smem_u32(&bar_full[st]), round & 1, abort_flag);
      if (!got && !*abort_flag) { *abort_flag = 1; if (P.status) atomicCAS(P.status, 0, 12); }
      got = __all_sync(0xffffffffu, got);
      if (!got) break;
      uint8_t* stage = smem + st * kStage + box * THB_AT_BOX_BYTES;
#pragma unroll
      for (int k = 0; k < kChunks; ++k) {
        const uint32_t ch = (uint32_t)(kChunks * half + k);
        float4 v[3];
#pragma unroll
        for (int q = 0; q < NT; ++q) {
          v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (q >= kFirstLoaded) {
            const uint8_t* b = stage + q * THB_AT_OPERAND_BYTES;
            if ((P.colmajor >> q) & 1) {
              float e[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t cl = 4u * ch + (uint32_t)j;
                e[j] = *reinterpret_cast<const float*>(b + cl * 128u + ((col_chunk ^ (cl & 7u)) << 4) + col_in);
              }
              v[q] = make_float4(e[0], e[1], e[2], e[3]);
            } else {
              v[q] = *reinterpret_cast<const float4*>(b + row_base + ((ch ^ row_xor) << 4));
            }
          }
        }
        float4& o = v[0];
        const float4& x = v[NT >= 2 ? 1 : 0];
        const float4& y = v[NT >= 3 ? 2 : 0];
        Op::apply(&o.x, &x.x, &y.x, s.val1, s.val2, &p1, &p2);
        Op::apply(&o.y, &x.y, &y.y, s.val1, s.val2, &p1, &p2);
        Op::apply(&o.z, &x.z, &y.z, s.val1, s.val2, &p1, &p2);
        Op::apply(&o.w, &x.w, &y.w, s.val1, s.val2, &p1, &p2);
        if (P.colmajor & 1) {
          const float e[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t cl = 4u * ch + (uint32_t)j;
            *reinterpret_cast<float*>(stage + cl * 128u + ((col_chunk ^ (cl & 7u)) << 4) + col_in) = e[j];
          }
        } else {
          *reinterpret_cast<float4*>(stage + row_base + ((ch ^ row_xor) << 4)) = o;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // results visible to the TMA unit
      __syncwarp();
      if (lane == 0) thb_mbar_arrive(thb_smem_u32(&bar_done[st]));
    }
  }
  __syncthreads();
}
