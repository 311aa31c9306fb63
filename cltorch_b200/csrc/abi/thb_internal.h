// Host-side declarations shared by the sources behind include/thb200.h.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <vector>
#include "thb200.h"

namespace thb {

// Records the message for thb200_last_error() and returns a non-zero status.
int fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
int fail_cuda(cudaError_t e, const char* what);

#define THB_CUDA(expr)                                         \
  do {                                                         \
    cudaError_t thb_e_ = (expr);                               \
    if (thb_e_ != cudaSuccess) return ::thb::fail_cuda(thb_e_, #expr); \
  } while (0)

// Per-call device timing (thb200_timing_*): when switched on, an entry point brackets what it
// enqueues with two CUDA events on its stream; thb200_timing_report resolves them. Off by default:
// the object then does nothing (no event is created, nothing is recorded).
struct CallTimer {
  CallTimer(void* stream, const char* name);
  ~CallTimer();
  cudaEvent_t start_ = nullptr, stop_ = nullptr;
  cudaStream_t stream_ = nullptr;
  const char* name_ = nullptr;
};
#define THB_TIMED(stream, name) ::thb::CallTimer thb_call_timer_((stream), (name))

struct Collapsed {
  int dims = 0;
  int64_t size[THB200_MAX_DIMS];
  int64_t stride[THB200_MAX_DIMS];
  bool contiguous() const { return dims == 1 && stride[0] == 1; }
};

int64_t num_elements(const thb200_tensor& t);  // 0 for ndim == 0, as THClTensor_nElement
bool collapse(int ndim, const int64_t* size, const int64_t* stride, int reduce_dim, Collapsed* out);
bool can_use_32bit(int ndim, const int64_t* size, const int64_t* stride);
int sm_count();  // of the current device, cached per device

// Order heuristic of the streaming kernels (thb_common.cpp): whether the contiguous operands `ptrs`
// (`bytes` each) should be walked from their end, given where the previous streaming kernel on this device
// stopped; and the note a kernel leaves for the next one.
bool stream_prefers_descending(const void* const* ptrs, int n, size_t bytes);
void stream_note_end(const void* const* ptrs, int n, size_t bytes, bool descending);
// The streaming kernels keep their grid-stride loops but are launched with one batch per block up
// to this bound (the largest gridDim.x): on B200 a block per batch, handed out by the hardware
// scheduler, measured 3-10% faster than a grid of 32 blocks per SM looping over the batches.
constexpr int64_t kMaxGridBlocks = 0x7fffffff;

// cuTensorMapEncodeTiled obtained through the runtime (PFN_cuTensorMapEncodeTiled_v12000 as void*),
// so that the library does not link libcuda; nullptr if the driver does not offer it.
void* tensor_map_encoder_ptr();

// Counter of finished blocks for a single-launch whole-tensor reduction (ThbFinish::ticket): zero
// between launches (the last block of a launch resets it). Launches take the library's 64 counters
// per device in turn; only a few such grids (592 blocks each) can be resident at a time, so a
// counter is never shared by two running launches. nullptr if the counters cannot be addressed.
unsigned int* reduce_ticket();

// Device int of the current device into which the kernels of one family with bounded waits store
// a non-zero code when a wait gives up (read and cleared by thb200_kernel_status, which reports
// family and code); nullptr on failure. One word per family, so that a report names the kind of
// launch that gave up.
enum StatusFamily {
  STATUS_STRIP_REDUCE = 1,   // sum / prod / moments over a strided dimension (TMA strips)
  STATUS_STRIP_ARGREDUCE = 2,  // max / min with indices over a strided dimension
  STATUS_STRIP_SCAN = 3,     // cumsum / cumprod over a strided dimension
  STATUS_STRIP_GEMV = 4,     // matrix-vector product over the columns of a row-major matrix
  STATUS_TILE_APPLY = 5,     // pointwise operators on large transposed operands (TMA tiles)
  STATUS_SELFTEST = 6,       // thb200_selftest_wait_expiry
  STATUS_EXCHANGE = 7,       // the wait for the other GPUs' partial results (thb200_exchange_fold)
  STATUS_FAMILIES = 8
};
int* device_status_word(int family);

// thb200_reduce_all with the cross-GPU push (push_cells == nullptr: plain reduction), and the launch of
// the bounded wait + fold over this GPU's cells; both live with the reduction kernels.
int reduce_all_impl(void* stream, int modify, int reduce, const thb200_tensor* in, float init, float mod_param,
                    const float* mod_point, int fin, float fin_param, float* d_out, float* scratch, size_t scratch_bytes,
                    unsigned long long* const* push_cells, int push_count, unsigned int push_epoch);
int exchange_fold_launch(void* stream, int reduce, const unsigned long long* cells, int count, unsigned int epoch,
                         float* d_out, unsigned long long limit_ns);
float exchange_identity(int reduce);

// Number of chunks to cut a reduced / scanned dimension of `rsize` elements into when only
// `threads` worker threads (blocks of 256, `blocks_per_sm` resident) exist per chunk: as many
// as fit one wave of resident blocks, 1 when the threads alone fill half the GPU.
uint32_t pick_chunks(int64_t threads, int64_t rsize, int blocks_per_sm);

// Kernel handles of one pointwise operator: device function pointers usable
// with cudaLaunchKernel (nvcc-compiled symbols or cudaKernel_t from NVRTC).
struct ApplyKernels {
  const void* contig = nullptr;
  const void* strided = nullptr;
  const void* tile2d = nullptr;
  const void* tile2d_v4 = nullptr;
  const void* tile_tma = nullptr;  // thb_apply_tile_tma; absent for run-time compiled expressions
  const void* rows2d = nullptr;
  int nt = 0;
  bool reads_out = true;
  const char* name = nullptr;
  const char* body = nullptr;
};

enum ApplyPlan { PLAN_NONE = 0, PLAN_CONTIG = 1, PLAN_STRIDED = 2, PLAN_TILE2D = 3, PLAN_ROWS2D = 4 };

// Chooses the kernel for these operands and launches it.
int launch_apply(const ApplyKernels& k, cudaStream_t st, int nt, const thb200_tensor* t, float val1,
                 float val2, const float* p1, const float* p2, bool dry_run, int* plan_out);

const ApplyKernels* builtin_op(int code);
int builtin_op_count();

// NVRTC: kernels for a user expression body, compiled on first use.
int expr_kernels(int nt, const std::string& body, const ApplyKernels** out);

}  // namespace thb
