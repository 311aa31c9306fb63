// mbarrier and TMA helpers shared by the GEMM, the strip pipelines and the TMA tile apply.
//
// FREESTANDING when compiled by NVRTC (the text is handed to it together with the apply
// kernels): no #include there, the few types it needs are declared below. Every wait on an
// mbarrier goes through thb_mbar_wait, which gives up after THB_GEMM_WAIT_LIMIT_NS.
#pragma once
#ifdef __CUDACC_RTC__
typedef unsigned char uint8_t;
typedef unsigned int uint32_t;
typedef unsigned long long uint64_t;
typedef unsigned long long uintptr_t;
// same size and alignment as the driver API's opaque tensor map (cuda.h)
struct alignas(64) CUtensorMap_st { unsigned long long opaque[16]; };
typedef CUtensorMap_st CUtensorMap;
#else
#include <cuda.h>
#include <stdint.h>
#endif

#define THB_GEMM_WAIT_LIMIT_NS 2000000000ull  // 2 s

__device__ __forceinline__ uint32_t thb_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void thb_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void thb_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool thb_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false when the limit ran out or another thread already gave up.
__device__ __forceinline__ unsigned long long thb_globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool thb_mbar_wait_ns(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                 unsigned long long limit_ns) {
  if (thb_mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = thb_globaltimer_ns();
  for (uint32_t i = 1;; ++i) {
    if (thb_mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0) {
      if (*abort_flag) return false;
      if (thb_globaltimer_ns() - t0 > limit_ns) return false;
    }
  }
}
__device__ __forceinline__ bool thb_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return thb_mbar_wait_ns(bar, parity, abort_flag, THB_GEMM_WAIT_LIMIT_NS);
}
__device__ __forceinline__ void thb_tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void thb_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrival on the barrier at the same shared-memory offset in CTA `cta_rank` of this thread-block cluster.
__device__ __forceinline__ void thb_mbar_arrive_cluster(uint32_t bar, uint32_t cta_rank) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t}"
      ::"r"(bar), "r"(cta_rank)
      : "memory");
}
// The same without release semantics: for hand-overs whose ordering comes from tcgen05 fences (tensor
// memory), so that the arrival does not wait for the thread's earlier global stores.
__device__ __forceinline__ void thb_mbar_arrive_cluster_relaxed(uint32_t bar, uint32_t cta_rank) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [remote];\n\t}"
      ::"r"(bar), "r"(cta_rank)
      : "memory");
}
__device__ __forceinline__ void thb_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void thb_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void thb_tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y)
               : "memory");
}
