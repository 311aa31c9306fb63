// Cross-GPU exchange of one float per GPU (include/thb200.h, thb200_exchange_*): each GPU's
// whole-tensor reduction stores its result straight into a cell in the memory of every GPU of
// the group (plain 8-byte stores over NVLink, issued by the reduction kernel's finishing block),
// and a one-block kernel on each GPU waits - bounded - for its own cells and folds them in rank
// order. No collective library, no host synchronisation, nothing reads a peer's memory.
#include "thb_internal.h"

#include <cstring>
#include <unistd.h>
#include <vector>

namespace {

const uint32_t kMagic = 0x78423230u;  // "xB20"

struct Handle {  // what a rank publishes; THB200_EXCHANGE_HANDLE_BYTES bytes
  uint32_t magic;
  int32_t pid, device, world, rank;
  uint32_t pad;
  uint64_t base;  // address of the cells in the owner's address space
  cudaIpcMemHandle_t ipc;
};
static_assert(sizeof(Handle) <= THB200_EXCHANGE_HANDLE_BYTES, "handle size");

}  // namespace

// Cells of one GPU: cell[parity][rank], parity = epoch & 1 (a rank may already be storing epoch e + 1
// while this GPU has not folded epoch e yet; it cannot reach e + 2 before, because its own fold of
// e + 1 needs this GPU's store of e + 1, which follows this GPU's fold of e in stream order).
struct thb200_exchange {
  int rank = 0, world = 0, device = 0;
  unsigned int epoch = 0;
  bool connected = false;
  unsigned long long* cells = nullptr;       // device, [2][world], this GPU's own
  float* local = nullptr;                    // device, this GPU's partial (also pushed to its own cell)
  unsigned long long** d_targets = nullptr;  // device, [2][world]: the cell (parity, this rank) in every GPU's buffer
  std::vector<void*> opened;                 // IPC mappings to close
};

using namespace thb;

extern "C" {

int thb200_exchange_create(int rank, int world, thb200_exchange** out, void* handle_out) {
  if (!out || !handle_out) return fail("exchange: null argument");
  if (world < 1 || world > 1024 || rank < 0 || rank >= world) return fail("exchange: rank %d outside a group of %d (at most 1024)", rank, world);
  thb200_exchange* x = new thb200_exchange();
  x->rank = rank;
  x->world = world;
  THB_CUDA(cudaGetDevice(&x->device));
  const size_t cell_bytes = sizeof(unsigned long long) * 2 * (size_t)world;
  // one allocation: cells, then the local partial (cudaMalloc, not a pool: it has to be exportable)
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, cell_bytes + 256);
  if (e != cudaSuccess) { delete x; return fail_cuda(e, "cudaMalloc(exchange cells)"); }
  x->cells = (unsigned long long*)p;
  x->local = (float*)((char*)p + cell_bytes);
  THB_CUDA(cudaMemset(p, 0, cell_bytes + 256));  // epoch 0 = nothing has arrived
  THB_CUDA(cudaMalloc((void**)&x->d_targets, sizeof(void*) * 2 * (size_t)world));
  Handle h;
  memset(&h, 0, sizeof h);
  h.magic = kMagic;
  h.pid = (int32_t)getpid();
  h.device = x->device;
  h.world = world;
  h.rank = rank;
  h.base = (uint64_t)(uintptr_t)x->cells;
  e = cudaIpcGetMemHandle(&h.ipc, x->cells);
  if (e != cudaSuccess) {
    // same-process groups do not need it; a process that cannot export still works with peers in its own process
    cudaGetLastError();
    memset(&h.ipc, 0, sizeof h.ipc);
  }
  memset(handle_out, 0, THB200_EXCHANGE_HANDLE_BYTES);
  memcpy(handle_out, &h, sizeof h);
  *out = x;
  return 0;
}

int thb200_exchange_connect(thb200_exchange* x, const void* all_handles) {
  if (!x || !all_handles) return fail("exchange: null argument");
  if (x->connected) return fail("exchange: already connected");
  int dev = -1;
  THB_CUDA(cudaGetDevice(&dev));
  if (dev != x->device) return fail("exchange: created on device %d, connect called with device %d current", x->device, dev);
  std::vector<unsigned long long*> targets(2 * (size_t)x->world);
  for (int j = 0; j < x->world; ++j) {
    Handle h;
    memcpy(&h, (const char*)all_handles + (size_t)j * THB200_EXCHANGE_HANDLE_BYTES, sizeof h);
    if (h.magic != kMagic || h.world != x->world || h.rank != j)
      return fail("exchange: handle %d is not the handle of rank %d in a group of %d", j, j, x->world);
    unsigned long long* base = nullptr;
    if (j == x->rank) {
      base = x->cells;
    } else if (h.pid == (int32_t)getpid()) {
      base = (unsigned long long*)(uintptr_t)h.base;  // same address space
      if (h.device != x->device) {
        int can = 0;
        THB_CUDA(cudaDeviceCanAccessPeer(&can, x->device, h.device));
        if (!can) return fail("exchange: device %d cannot store to device %d", x->device, h.device);
        cudaError_t e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail_cuda(e, "cudaDeviceEnablePeerAccess");
        cudaGetLastError();
      }
    } else {
      void* p = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&p, h.ipc, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) return fail_cuda(e, "cudaIpcOpenMemHandle (peer buffer of the exchange)");
      x->opened.push_back(p);
      base = (unsigned long long*)p;
    }
    for (int parity = 0; parity < 2; ++parity) targets[(size_t)parity * x->world + j] = base + (size_t)parity * x->world + x->rank;
  }
  THB_CUDA(cudaMemcpy(x->d_targets, targets.data(), sizeof(void*) * targets.size(), cudaMemcpyHostToDevice));
  x->connected = true;
  return 0;
}

int thb200_exchange_push(void* stream, thb200_exchange* x, int reduce, const thb200_tensor* in, float* scratch, size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_exchange_push");
  if (!x || !x->connected) return fail("exchange: not connected");
  const unsigned int epoch = x->epoch + 1;
  const int parity = (int)(epoch & 1u);
  int rc = reduce_all_impl(stream, THB200_MOD_COPY, reduce, in, exchange_identity(reduce), 0.f, nullptr, THB200_FIN_NONE, 1.f, x->local,
                           scratch, scratch_bytes, x->d_targets + (size_t)parity * x->world, x->world, epoch);
  if (rc == 0) x->epoch = epoch;
  return rc;
}

int thb200_exchange_fold(void* stream, thb200_exchange* x, int reduce, float* d_out, uint64_t wait_limit_ns) {
  THB_TIMED(stream, "thb200_exchange_fold");
  if (!x || !x->connected) return fail("exchange: not connected");
  if (!d_out) return fail("exchange: null result pointer");
  if (x->epoch == 0) return fail("exchange: fold before the first push");
  if (wait_limit_ns == 0 || wait_limit_ns > 60000000000ull) return fail("exchange: the wait limit must be between 1 ns and 60 s");
  const int parity = (int)(x->epoch & 1u);
  return exchange_fold_launch(stream, reduce, x->cells + (size_t)parity * x->world, x->world, x->epoch, d_out, wait_limit_ns);
}

int thb200_exchange_reduce(void* stream, thb200_exchange* x, int reduce, const thb200_tensor* in, float* d_out, float* scratch,
                           size_t scratch_bytes, uint64_t wait_limit_ns) {
  if (int rc = thb200_exchange_push(stream, x, reduce, in, scratch, scratch_bytes)) return rc;
  return thb200_exchange_fold(stream, x, reduce, d_out, wait_limit_ns);
}

int thb200_exchange_destroy(thb200_exchange* x) {
  if (!x) return 0;
  for (void* p : x->opened) cudaIpcCloseMemHandle(p);
  if (x->d_targets) cudaFree(x->d_targets);
  if (x->cells) cudaFree(x->cells);
  cudaGetLastError();
  delete x;
  return 0;
}

}  // extern "C"
