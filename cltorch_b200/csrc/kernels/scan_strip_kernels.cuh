// Single-pass scan along a non-innermost dimension when the other dimensions are too
// small for one thread per column to keep HBM busy: the matrix is cut into strips of 128
// columns, one CTA walks a strip from the first row to the last, and a TMA pipeline of
// 8 x (32 rows x 512 bytes) keeps 128 KB of loads in flight per CTA, so that a hundred or
// so CTAs saturate HBM with 8 bytes of traffic per element (the chunked alternative,
// thb_scan_cols in three phases, moves 12).
//
// Same job as THClTensor_kernel_scanOuterDim (reference src/lib/THClTensorMathScan.cl:27-50).
//
// Warp 0 lane 0 issues the loads (cp.async.bulk.tensor.3d, no multicast), warps 1-4 hold one
// column per thread: they add up the 32 values of a stage in double and write the running
// values back into the stage, which warp 5 hands to the TMA unit as one store of 32 rows x 512
// bytes (no thread stores to global memory). Every wait is bounded (THB_GEMM_WAIT_LIMIT_NS); on
// expiry the waiter writes *status and everybody leaves.
#pragma once
#include "gemm_kernels.cuh"  // mbarrier / TMA helpers
#include "scan_kernels.cuh"

#define THB_SS_COLS 128
#define THB_SS_ROWS 32
#define THB_SS_STAGES 8  // 12 measured 3-8 % slower on the reductions, 2 % faster on the scan
#define THB_SS_THREADS 160
#define THB_SS_STAGE_BYTES (THB_SS_ROWS * THB_SS_COLS * 4)
#define THB_SS_SMEM (THB_SS_STAGES * THB_SS_STAGE_BYTES + 128 /*alignment*/ + 512 /*barriers: up to 3 per stage, and two flags*/ + \
                     THB_SS_STAGES * THB_SS_ROWS * 8 /*row weights of the matrix-vector consumer*/)

#define THB_SCAN_STRIP_THREADS 192  // warp 0 loads, warps 1-4 scan, warp 5 stores

__device__ __forceinline__ void thb_tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}

template <class Op>
__global__ void __launch_bounds__(THB_SCAN_STRIP_THREADS, 1)
thb_scan_strips(const __grid_constant__ CUtensorMap map_src, const __grid_constant__ CUtensorMap map_dst, thb_u32 n,
                thb_i64 inner, int strips_per_outer, int total_strips, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  uint64_t* bar_full = (uint64_t*)(smem + THB_SS_STAGES * THB_SS_STAGE_BYTES);
  uint64_t* bar_empty = bar_full + THB_SS_STAGES;
  uint64_t* bar_done = bar_empty + THB_SS_STAGES;
  volatile int* abort_flag = (volatile int*)(bar_done + THB_SS_STAGES);
  volatile int* never_set = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < THB_SS_STAGES; ++s) {
      thb_mbar_init(thb_smem_u32(&bar_full[s]), 1);
      thb_mbar_init(thb_smem_u32(&bar_empty[s]), 1);  // the store warp, once the store has read the stage
      thb_mbar_init(thb_smem_u32(&bar_done[s]), 4);   // one arrival per scanning warp
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int row_blocks = (int)((n + THB_SS_ROWS - 1) / THB_SS_ROWS);

  if (warp == 0) {
    if (lane == 0) {
      long long it = 0;
      bool ok = true;
      for (int strip = blockIdx.x; strip < total_strips && ok; strip += gridDim.x) {
        const int o = strip / strips_per_outer;
        const int c0 = (strip - o * strips_per_outer) * THB_SS_COLS;
        for (int rb = 0; rb < row_blocks; ++rb, ++it) {
          const int s = (int)(it % THB_SS_STAGES);
          const uint32_t round = (uint32_t)(it / THB_SS_STAGES);
          if (it >= THB_SS_STAGES && !thb_mbar_wait(thb_smem_u32(&bar_empty[s]), (round - 1) & 1, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; if (status) atomicCAS(status, 0, 1); }
            ok = false;
            break;
          }
          const uint32_t full = thb_smem_u32(&bar_full[s]);
          thb_mbar_expect_tx(full, THB_SS_STAGE_BYTES);  // rows or columns past the edge arrive as zeros
          thb_tma_load_3d(thb_smem_u32(smem + s * THB_SS_STAGE_BYTES), &map_src, full, c0, rb * THB_SS_ROWS, o);
        }
      }
      if (*abort_flag) {
        // do not leave while copies into this CTA's shared memory are in flight
        for (long long j = (it > THB_SS_STAGES ? it - THB_SS_STAGES : 0); j < it; ++j)
          thb_mbar_wait(thb_smem_u32(&bar_full[j % THB_SS_STAGES]), (uint32_t)(j / THB_SS_STAGES) & 1, never_set);
      }
    }
  } else if (warp == 5) {
    // The scanned stage goes back as one box of 32 rows x 512 bytes; what lies past the last row
    // or column of the matrix is clipped by the TMA unit.
    if (lane == 0) {
      long long it = 0;
      bool ok = true;
      for (int strip = blockIdx.x; strip < total_strips && ok; strip += gridDim.x) {
        const int o = strip / strips_per_outer;
        const int c0 = (strip - o * strips_per_outer) * THB_SS_COLS;
        for (int rb = 0; rb < row_blocks; ++rb, ++it) {
          const int s = (int)(it % THB_SS_STAGES);
          const uint32_t round = (uint32_t)(it / THB_SS_STAGES);
          if (!thb_mbar_wait(thb_smem_u32(&bar_done[s]), round & 1, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; if (status) atomicCAS(status, 0, 3); }
            ok = false;
            break;
          }
          thb_tma_store_3d(&map_dst, thb_smem_u32(smem + s * THB_SS_STAGE_BYTES), c0, rb * THB_SS_ROWS, o);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          thb_mbar_arrive(thb_smem_u32(&bar_empty[s]));
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else {
    const int tx = threadIdx.x - 32;  // 0..127: the column of the strip
    long long it = 0;
    bool ok = true;
    for (int strip = blockIdx.x; strip < total_strips && ok; strip += gridDim.x) {
      double acc = Op::identity();
      for (int rb = 0; rb < row_blocks; ++rb, ++it) {
        const int s = (int)(it % THB_SS_STAGES);
        const uint32_t round = (uint32_t)(it / THB_SS_STAGES);
        bool got = thb_mbar_wait(thb_smem_u32(&bar_full[s]), round & 1, abort_flag);
        if (!got && !*abort_flag) { *abort_flag = 1; if (status) atomicCAS(status, 0, 2); }
        got = __all_sync(0xffffffffu, got);
        if (!got) { ok = false; break; }
        float* tile = reinterpret_cast<float*>(smem + s * THB_SS_STAGE_BYTES) + tx;
        float v[THB_SS_ROWS];
#pragma unroll
        for (int r = 0; r < THB_SS_ROWS; ++r) v[r] = tile[r * THB_SS_COLS];
        // rows past the end hold zeros and are never stored; the running value is not used after them
#pragma unroll
        for (int r = 0; r < THB_SS_ROWS; ++r) {
          acc = Op::apply(acc, (double)v[r]);
          tile[r * THB_SS_COLS] = (float)acc;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // results visible to the TMA unit
        __syncwarp();
        if (lane == 0) thb_mbar_arrive(thb_smem_u32(&bar_done[s]));
      }
    }
  }
  __syncthreads();
}
