// State, per-device contexts and the error convention of include/THCl.h.
#include "thcl_internal.h"
#include <atomic>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace thcl {

static thread_local int g_depth = 0;
static thread_local std::string g_last_error;
static THClErrorHandler g_handler = nullptr;
static void* g_handler_data = nullptr;

Scope::Scope() {
  if (g_depth++ == 0) g_last_error.clear();
}
Scope::~Scope() { --g_depth; }
int Scope::depth() { return g_depth; }

void raise(const char* fmt, ...) {
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  throw Error(buf);
}

void arg_check(bool cond, int arg, const char* msg) {
  if (!cond) raise("bad argument #%d: %s", arg, msg);
}

void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) raise("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

void check_thb(int rc) {
  if (rc != 0) raise("%s", thb200_last_error());
}

void report(const char* msg) {
  g_last_error = msg;
  if (g_handler) {
    g_handler(msg, g_handler_data);
    return;
  }
  // default, as Torch7's default error handler: no way to continue
  fprintf(stderr, "THCl error: %s\n", msg);
  abort();
}

void clear_error() { g_last_error.clear(); }

void use_device(int device) {
  int cur = -1;
  check_cuda(cudaGetDevice(&cur), "cudaGetDevice");
  if (cur != device) check_cuda(cudaSetDevice(device), "cudaSetDevice");
}

THClDeviceContext* context(THClState* state, int device) {
  if (!state) raise("null THClState");
  if (!state->initialized) THCl_initializeState(state);
  if (device < 0 || device >= state->allocatedDevices)
    raise("Please select a device between 1 and %d (got %d)", state->allocatedDevices, device + 1);
  THClDeviceContext*& ctx = state->contextByDevice[device];
  if (!ctx) {
    use_device(device);
    ctx = new THClDeviceContext();
    ctx->device = device;
    check_cuda(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    ctx->owns_stream = true;
    check_cuda(cudaMalloc((void**)&ctx->result, 64 * sizeof(float)), "cudaMalloc(result)");
    check_cuda(cudaMemset(ctx->result, 0, 64 * sizeof(float)), "cudaMemset(result)");
    check_cuda(cudaMallocHost((void**)&ctx->result_host, 64 * sizeof(float)), "cudaMallocHost(result)");
    memset(ctx->result_host, 0, 64 * sizeof(float));
    void* mapped = nullptr;
    if (cudaHostGetDevicePointer(&mapped, ctx->result_host, 0) == cudaSuccess) ctx->result_mapped = (float*)mapped;
    else cudaGetLastError();
    ctx->scratch_bytes = 4u << 20;
    check_cuda(cudaMalloc((void**)&ctx->scratch, ctx->scratch_bytes), "cudaMalloc(scratch)");
    // keep freed storage memory in the stream-ordered pool instead of returning it at every sync
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
      unsigned long long keep = ~0ull;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    ctx->scratch_space.wrapper = ctx->result;
    ctx->scratch_space.data = ctx->result_host;
    state->scratchSpaceByDevice[device] = &ctx->scratch_space;
    if (state->trace) printf("THCl: created context for device %d\n", device);
  }
  return ctx;
}

float* ensure_scratch(THClDeviceContext* ctx, size_t bytes) {
  if (bytes > ctx->scratch_bytes) {
    use_device(ctx->device);
    // cudaFree waits for the work that may still read the old buffer
    check_cuda(cudaFree(ctx->scratch), "cudaFree(scratch)");
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = bytes + bytes / 4;
    check_cuda(cudaMalloc((void**)&ctx->scratch, want), "cudaMalloc(scratch)");
    ctx->scratch_bytes = want;
  }
  return ctx->scratch;
}

void* ensure_gemm_ws(THClDeviceContext* ctx, size_t bytes) {
  if (bytes > ctx->gemm_ws_bytes) {
    use_device(ctx->device);
    if (ctx->gemm_ws) check_cuda(cudaFree(ctx->gemm_ws), "cudaFree(gemm workspace)");
    ctx->gemm_ws = nullptr;
    ctx->gemm_ws_bytes = 0;
    check_cuda(cudaMalloc(&ctx->gemm_ws, bytes), "cudaMalloc(gemm workspace)");
    ctx->gemm_ws_bytes = bytes;
  }
  return ctx->gemm_ws;
}

void sync_stream(THClDeviceContext* ctx) {
  check_cuda(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
  if (ctx->gemm_pending) {
    ctx->gemm_pending = false;
    int st = thb200_gemm_status(ctx->stream, ctx->gemm_shape[0], ctx->gemm_shape[1], ctx->gemm_shape[2],
                                ctx->gemm_shape[3], ctx->gemm_ws);
    if (st != 0) raise("GEMM kernel did not complete: a bounded wait gave up (status %d); the result is undefined", st);
  }
  // kernels with bounded waits other than the GEMM report through the library's status word
  // (the query costs nothing when no such kernel ran since the last one)
  const int st = thb200_kernel_status(ctx->stream);
  if (st != 0) {
    static const char* const kFamily[] = {"?", "sum over a strided dimension", "max/min over a strided dimension", "scan",
                                          "matrix-vector product", "pointwise operator on transposed operands", "self-test",
                                          "exchange between GPUs (a rank is absent or late)"};
    raise("a kernel did not complete: a bounded wait gave up (%s, code %d); its result is undefined",
          st > 0 ? kFamily[(st >> 8) & 7] : "status unreadable", st > 0 ? (st & 255) : st);
  }
}

// A quiet NaN with a payload that no kernel of this library produces: "the result has not arrived".
static const uint32_t kResultPending = 0x7FC5A5A5u;

float* host_result_target(THClDeviceContext* ctx) {
  if (!ctx->result_mapped) return ctx->result;
  *reinterpret_cast<volatile uint32_t*>(ctx->result_host) = kResultPending;
  return ctx->result_mapped;
}

float read_host_result(THClDeviceContext* ctx, int slot) {
  if (!ctx->result_mapped || slot != 0 || ctx->gemm_pending) {
    if (!ctx->result_mapped)
      check_cuda(cudaMemcpyAsync(ctx->result_host + slot, ctx->result + slot, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream),
                 "cudaMemcpyAsync");
    sync_stream(ctx);
    return ctx->result_host[slot];
  }
  // The kernel stores its one result straight into this pinned word. Watching the word costs a few
  // microseconds less than a stream synchronisation, which returns only after the kernel has been
  // retired. Every so often the stream is asked whether it is done, so that a result that happens
  // to equal the marker, or a launch that failed, cannot keep the host here.
  volatile uint32_t* word = reinterpret_cast<volatile uint32_t*>(ctx->result_host);
  for (unsigned spin = 1; *word == kResultPending; ++spin) {
    if ((spin & 2047u) == 0) {
      cudaError_t q = cudaStreamQuery(ctx->stream);
      if (q == cudaSuccess) break;
      if (q != cudaErrorNotReady) check_cuda(q, "cudaStreamQuery");
    }
  }
  std::atomic_thread_fence(std::memory_order_acquire);
  // bounded-wait status words are read at the next full synchronisation
  return ctx->result_host[0];
}

void after_launch(THClState* state, THClDeviceContext* ctx) {
  if (state->addFinish) sync_stream(ctx);
}

}  // namespace thcl

using namespace thcl;

extern "C" {

void THClSetErrorHandler(THClErrorHandler handler, void* data) {
  g_handler = handler;
  g_handler_data = data;
}
const char* THClLastError(void) { return g_last_error.c_str(); }
void THClClearError(void) { g_last_error.clear(); }

void THClInit(THClState* state) {
  memset(state, 0, sizeof *state);
}

void THCl_initializeState(THClState* state) {
  THCL_BEGIN
  if (state->initialized) return;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0)
    raise("no CUDA device available (%s): this backend has no CPU path", e != cudaSuccess ? cudaGetErrorString(e) : "0 devices");
  state->allocatedDevices = n;
  state->currentDevice = 0;
  state->scratchSpaceByDevice = (THClScratchSpace**)calloc(n, sizeof(THClScratchSpace*));
  state->contextByDevice = (THClDeviceContext**)calloc(n, sizeof(THClDeviceContext*));
  state->initialized = 1;
  THCL_END_VOID
}

void THClShutdown(THClState* state) {
  THCL_BEGIN
  if (!state->initialized) return;
  for (int d = 0; d < state->allocatedDevices; ++d) {
    THClDeviceContext* ctx = state->contextByDevice[d];
    if (!ctx) continue;
    use_device(d);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->result);
    cudaFreeHost(ctx->result_host);
    cudaFree(ctx->scratch);
    if (ctx->gemm_ws) cudaFree(ctx->gemm_ws);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
  }
  free(state->scratchSpaceByDevice);
  free(state->contextByDevice);
  memset(state, 0, sizeof *state);
  THCL_END_VOID
}

void THClSetAllowNonGpus(THClState* state, int allowNonGpus) { state->allowNonGpus = allowNonGpus; }

int THClState_getNumDevices(THClState* state) {
  THCL_BEGIN
  if (!state->initialized) THCl_initializeState(state);
  return state->allocatedDevices;
  THCL_END(0)
}

void THClState_setDevice(THClState* state, int device) {
  THCL_BEGIN
  context(state, device);
  state->currentDevice = device;
  use_device(device);
  THCL_END_VOID
}

int THClState_getDevice(THClState* state) { return state->currentDevice; }

struct THClScratchSpace* THClState_getDeviceScratchSpace(THClState* state, int device, int stream) {
  THCL_BEGIN
  if (stream != 0) raise("stream %d not available", stream);
  return &context(state, device)->scratch_space;
  THCL_END(nullptr)
}

size_t THClState_getDeviceScratchSpaceSize(THClState*, int) { return 64 * sizeof(float); }

struct THClScratchSpace* THClState_getCurrentDeviceScratchSpace(THClState* state) {
  return THClState_getDeviceScratchSpace(state, state->currentDevice, 0);
}

size_t THClState_getCurrentDeviceScratchSpaceSize(THClState* state) {
  return THClState_getDeviceScratchSpaceSize(state, state->currentDevice);
}

void THClSynchronize(THClState* state) {
  THCL_BEGIN
  THClDeviceContext* ctx = context(state, state->currentDevice);
  use_device(ctx->device);
  sync_stream(ctx);
  THCL_END_VOID
}

void* THClState_getStream(THClState* state, int device) {
  THCL_BEGIN
  return (void*)context(state, device)->stream;
  THCL_END(nullptr)
}

void THClState_setStream(THClState* state, int device, void* stream) {
  THCL_BEGIN
  THClDeviceContext* ctx = context(state, device);
  use_device(device);
  check_cuda(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
  if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
  ctx->stream = (cudaStream_t)stream;
  ctx->owns_stream = false;
  THCL_END_VOID
}

}  // extern "C"
