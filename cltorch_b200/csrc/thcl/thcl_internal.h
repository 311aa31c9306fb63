// Internals of the THCl-shaped host layer (include/THCl.h).
#pragma once
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>
#include <vector>

#include "THCl.h"
#include "thb200.h"

struct THClDeviceContext {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  float* result = nullptr;        // 64 device floats: results of host-scalar reductions
  float* result_host = nullptr;   // pinned mirror of `result`
  float* result_mapped = nullptr; // device address of `result_host` when kernels can write there directly, else null
  float* scratch = nullptr;       // reduction partials
  size_t scratch_bytes = 0;
  void* gemm_ws = nullptr;        // split operands of the GEMM
  size_t gemm_ws_bytes = 0;
  bool gemm_pending = false;      // a GEMM was enqueued and its status word not read yet
  long gemm_shape[4] = {0, 0, 0, 0};
  THClScratchSpace scratch_space{nullptr, nullptr};
};

namespace thcl {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

[[noreturn]] void raise(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
void arg_check(bool cond, int arg, const char* msg);  // THArgCheck
void check_cuda(cudaError_t e, const char* what);
void check_thb(int rc);  // non-zero status of a thb200_* call -> Error with its message

// Error reporting at the C boundary: nested API calls rethrow, the outermost
// one runs the installed handler.
struct Scope {
  Scope();
  ~Scope();
  static int depth();
};
void report(const char* msg);
void clear_error();

#define THCL_BEGIN        \
  ::thcl::Scope thcl_scope_; \
  try {
#define THCL_END(ret)                         \
  }                                           \
  catch (const std::exception& e) {           \
    if (::thcl::Scope::depth() > 1) throw;    \
    ::thcl::report(e.what());                 \
    return ret;                               \
  }
#define THCL_END_VOID                         \
  }                                           \
  catch (const std::exception& e) {           \
    if (::thcl::Scope::depth() > 1) throw;    \
    ::thcl::report(e.what());                 \
    return;                                   \
  }

THClDeviceContext* context(THClState* state, int device);  // created on first use
void use_device(int device);                               // cudaSetDevice if needed
float* ensure_scratch(THClDeviceContext* ctx, size_t bytes);
void* ensure_gemm_ws(THClDeviceContext* ctx, size_t bytes);
void after_launch(THClState* state, THClDeviceContext* ctx);  // addFinish
// cudaStreamSynchronize, then the status word of the last GEMM if one is pending: a
// GEMM whose bounded waits gave up surfaces here as an error instead of silently
// leaving an undefined result.
void sync_stream(THClDeviceContext* ctx);

// View of a tensor for the thin ABI; keeps the int64 copies of size/stride alive.
struct View {
  thb200_tensor t;
  int64_t size[THB200_MAX_DIMS];
  int64_t stride[THB200_MAX_DIMS];
  View() { t.data = nullptr; t.ndim = 0; t.size = size; t.stride = stride; }
  View(const View&) = delete;
  void set(const THClTensor* x);
};

// Pointwise apply over 1..3 tensors with overlap handling
// (THClTensor_pointwiseApply, reference src/lib/THClApply.cpp:145-240).
// Exactly one of `op` (built-in name) and `expr` (rewritten body) is given.
void pointwise(THClState* state, int nt, THClTensor** tensors, const bool* read_write, const char* op,
               const char* expr, float val1, float val2, const THClTensor* point1);

// Where a reduction whose result the host wants at once puts it: straight into the pinned host
// buffer when the device can address it, else into the device buffer. Call it right before the
// launch that writes the result: it marks the pinned word as "not arrived yet".
float* host_result_target(THClDeviceContext* ctx);
// Returns slot `slot` of that target once the result has arrived: by watching the pinned word
// (slot 0, mapped buffer), else by synchronising the stream.
float read_host_result(THClDeviceContext* ctx, int slot);

}  // namespace thcl
