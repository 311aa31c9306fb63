/* thb200.h — the thin CUDA C ABI underneath the THCl-shaped host library.
 *
 * Plain pointers, sizes and strides only. Every device pointer is an ordinary
 * CUDA global-memory address on the current device; `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream). All launches
 * are asynchronous; nothing here synchronises the host except where stated.
 *
 * Return value: 0 on success, non-zero on failure, with the reason available
 * from thb200_last_error() (thread-local, valid until the next failing call on
 * the same thread).
 *
 * Each entry point names the interface of the reference (hughperkins/cltorch,
 * paths relative to its root) that it stands in for.
 */
#ifndef THB200_H
#define THB200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define THB200_MAX_DIMS 25 /* MAX_CLTORCH_DIMS, src/lib/THClReduceApplyUtils.h:19 */

/* A strided fp32 view. `data` addresses element (0,...,0), i.e. storage base +
 * storageOffset; `size`/`stride` are in elements, un-collapsed, row-major
 * meaning as in THClTensor (src/lib/THClTensor.h:14-27). ndim == 0 is a point
 * tensor / empty tensor: zero elements for apply, one float for the scalar
 * arguments named `point`. */
typedef struct thb200_tensor {
  float* data;
  int ndim;
  const int64_t* size;
  const int64_t* stride;
} thb200_tensor;

const char* thb200_last_error(void);

/* ---- host-side index helpers (no GPU needed) ------------------------------ */

/* TensorInfo<IndexType>::TensorInfo, src/lib/THClReduceApplyUtils.h:68-170:
 * drop size-1 dims, merge dim i into i+1 when stride[i] == size[i+1]*stride[i+1];
 * `reduce_dim` (or -1) is treated as size 1. Writes at most ndim entries to
 * out_size/out_stride and returns the collapsed dim count (>= 1), or -1. */
int thb200_collapse_dims(int ndim, const int64_t* size, const int64_t* stride, int reduce_dim,
                         int64_t* out_size, int64_t* out_stride);
/* THCL_canUse32BitIndexMath, src/lib/THClReduceApplyUtils.cpp:9-30. */
int thb200_can_use_32bit_index(int ndim, const int64_t* size, const int64_t* stride);
/* THCL_overlappingIndices, src/lib/THClReduceApplyUtils.cpp:69-121 (dims sorted
 * by ascending stride; the reference's qsort comparator is not a valid ordering). */
int thb200_overlapping_indices(int ndim, const int64_t* size, const int64_t* stride);
/* Which kernel thb200_apply_* would pick for these operands, without launching:
 * 0 = nothing to do, 1 = contiguous 128-bit, 2 = strided, 3 = 2-D tile (transposed
 * operands), 4 = 2-D rows (unit inner stride, 128-bit); < 0 = error. */
int thb200_apply_plan(int ntensors, const thb200_tensor* t);

/* ---- pointwise apply ------------------------------------------------------ */

/* Code of a built-in operator by name ("ADD_3", "MULC_1", ...; the list is
 * cltorch_b200/csrc/kernels/apply_ops.def), or -1. */
int thb200_op_code(const char* name);
/* Number of tensors a built-in operator takes (1..3), or -1. */
int thb200_op_arity(int op);

/* THClTensor_pointwiseApply1/2/3 with a built-in operator, src/lib/THClApply.cpp:145-287
 * and kernel src/lib/THClApply.cl:47-102. t[0] is the read/write operand. All
 * operands need equal element counts, not equal shapes. Overlapping read/write
 * operands are the caller's business (the THCl layer routes them through a
 * contiguous temporary as the reference does). */
int thb200_apply_op(void* stream, int op, int ntensors, const thb200_tensor* t,
                    float val1, float val2, const float* point1, const float* point2);

/* THClTensor_apply / _map / _map2 after the x,y,z rewrite,
 * src/lib/THClTensorMathPointwise.cpp:79-146: `body` is C code over *out, *in1,
 * *in2 (and val1, val2, *pointTensor1, *pointTensor2), compiled once per
 * (ntensors, body) with NVRTC for sm_100a and cached for the process. */
int thb200_apply_expr(void* stream, const char* body, int ntensors, const thb200_tensor* t,
                      float val1, float val2, const float* point1, const float* point2);
/* The x/y/z -> (*out)/(*in1)/(*in2) rewrite itself, token-wise; unsuffixed
 * floating literals get an `f`. Returns the length written (excluding NUL) or
 * -1 if `cap` is too small. */
int thb200_rewrite_expr(const char* expr, int ntensors, char* out, size_t cap);

/* ---- per-call device timing -------------------------------------------------
 * The thin equivalent of cltorch.setProfiling / dumpProfiling and setEnableTiming / dumpTimings
 * (src/init.cpp:130-178, EasyCL event profiling and StatefulTimer buckets): while switched on,
 * every entry point of this header that takes a stream brackets what it enqueues with two CUDA
 * events. thb200_timing_report waits for the outstanding events and writes one line per entry
 * point, "<name> <calls> <total milliseconds>", into buf (NUL-terminated, truncated to capacity);
 * it returns the size the whole report needs. Off by default; thb200_reduce_dim_noalloc is never
 * timed (events are driver allocations). */
void thb200_timing_enable(int on);
void thb200_timing_reset(void);
size_t thb200_timing_report(char* buf, size_t capacity);

/* ---- reductions ----------------------------------------------------------- */

enum thb200_modify { THB200_MOD_COPY = 0, THB200_MOD_ABSPOW = 1, THB200_MOD_NEZERO = 2, THB200_MOD_SQDEV = 3 };
enum thb200_reduce { THB200_RED_ADD = 0, THB200_RED_MUL = 1, THB200_RED_MIN = 2, THB200_RED_MAX = 3,
                     THB200_RED_AND = 4, THB200_RED_OR = 5 };
enum thb200_final { THB200_FIN_NONE = 0, THB200_FIN_DIV = 1, THB200_FIN_DIV_SQRT = 2 };

/* Bytes of scratch (global memory beyond input and output) that
 * thb200_reduce_all needs for `n` elements: one 8-byte partial per pass-1 block
 * (at most 592 blocks). Must be 8-byte aligned. */
size_t thb200_reduce_all_scratch_bytes(int64_t n);

/* THClTensor_reduceAll, src/lib/THClReduceAll.cpp:276-316 with kernels
 * src/lib/THClReduceAll.cl:24-100: r = init; r = reduce(r, modify(e)) over all
 * elements; *d_out = finalise(r). One launch: every block writes one partial into
 * `scratch`, then draws a ticket (the only atomic; data never goes through atomics);
 * the block that draws the last ticket folds all partials in a fixed order, so the
 * result does not depend on which block that is. The ticket is one of 64 counters per
 * device inside the library's device image, used in turn; a counter is zero between
 * launches (the last block resets it). Consequences: at most 64 whole-tensor
 * reductions may be in flight on a device at a time, replays of a captured graph that
 * contains one must not overlap each other, and after a launch that did not run to its
 * end (a sticky error) the counters are put back to zero by the next
 * thb200_kernel_status call that reports a failure. Sums and products accumulate in
 * double and round to fp32 once at the end.
 * `mod_param` is the exponent of ABSPOW; `mod_point` the device-resident mean of
 * SQDEV; `fin_param` the divisor of FIN_DIV / FIN_DIV_SQRT. d_out is a device
 * pointer: the result never visits the host (point tensors, README.md:88-138). */
int thb200_reduce_all(void* stream, int modify, int reduce, const thb200_tensor* in, float init,
                      float mod_param, const float* mod_point, int fin, float fin_param,
                      float* d_out, float* scratch, size_t scratch_bytes);

/* Reductions and scans over a non-innermost dimension of a contiguous tensor, matrix-vector
 * products and pointwise operators on large transposed operands stream through TMA pipelines
 * whose waits on shared-memory barriers are bounded (2 s). If such a wait ever gives up, the
 * kernel stores a non-zero code in the status word of its kernel family (inside the library's
 * device image) and leaves its output undefined. This call synchronises `stream`, returns
 * 256 * family + code of the first family whose word is set (0 = every kernel since the last call
 * completed) and clears all of them; < 0 if they cannot be read. Families: 1 sum / product /
 * moments over a strided dimension, 2 max / min with indices over a strided dimension, 3 scans,
 * 4 matrix-vector products, 5 pointwise operators on transposed operands, 6 the self-test below,
 * 7 the cross-GPU exchange (thb200_exchange_fold; code = 1 + first missing rank).
 * Codes: 1 = the producer's wait for a free stage, 2 = a consumer's wait for a full stage, other
 * values as the kernel documents. When no such kernel was launched on the current device since
 * the last call it returns 0 at once, without synchronising. */
int thb200_kernel_status(void* stream);

/* Runs the give-up path of those bounded waits on purpose, harmlessly: a one-warp kernel waits on
 * a shared-memory barrier that nothing arrives on (no copy is in flight), for at most `limit_ns`
 * nanoseconds (1 .. 1e9), then stores `code` (1 .. 255) in the status word of family 6 and returns.
 * thb200_kernel_status then reports 256 * 6 + code and the stream stays usable. For tests of a
 * host's error handling; no counterpart in the reference. */
int thb200_selftest_wait_expiry(void* stream, uint64_t limit_ns, int code);

/* ---- whole-tensor reduction over the GPUs of one box ------------------------
 * No counterpart in the reference (one OpenCL context per device, cross-device copy "Not
 * implemented", src/lib/THClTensorCopy.cpp:185-220). A tensor sharded over `world` GPUs, one
 * process (or thread) per GPU: every rank reduces its shard and all ranks end up with the same
 * total, device-resident, bit-identical (folded in rank order), without a collective library and
 * without a host synchronisation.
 *
 *   create   on each rank, with its GPU current: allocates this GPU's cells and fills a
 *            THB200_EXCHANGE_HANDLE_BYTES-byte handle.
 *   (the host passes every rank all handles, in rank order: MPI, torch.distributed, a file ...)
 *   connect  maps the other ranks' cells (CUDA IPC between processes, peer access within one).
 *   push     thb200_reduce_all of this rank's shard (modify = copy) in ONE launch whose finishing
 *            block also stores the result, tagged with the step number, into this rank's cell on
 *            every GPU: plain 8-byte stores over NVLink. It waits for nobody.
 *   fold     one block waits until this GPU's cells of all ranks carry the current step number and
 *            folds them in rank order into *d_out. The block may take its place while the kernel
 *            before it in the stream (this rank's push) is still running, so that it is watching
 *            when the last cell arrives; it writes only after that kernel has completed. The wait is
 *            bounded by wait_limit_ns, counted from the block's start (a rank that is absent or
 *            late; allow for this rank's own reduction): on expiry *d_out is NaN, the status word of family 7 gets
 *            1 + the first missing rank (see thb200_kernel_status) and the stream stays usable.
 *   reduce   push followed by fold.
 * push and fold of one step must be issued in that order on every rank, steps in the same order
 * on all ranks; `scratch` as for thb200_reduce_all. All ranks of one box must be able to store
 * to each other (NVLink / PCIe peer access). */
#define THB200_EXCHANGE_HANDLE_BYTES 128
typedef struct thb200_exchange thb200_exchange;
int thb200_exchange_create(int rank, int world, thb200_exchange** out, void* handle_out);
int thb200_exchange_connect(thb200_exchange* x, const void* all_handles);
int thb200_exchange_push(void* stream, thb200_exchange* x, int reduce, const thb200_tensor* in, float* scratch,
                         size_t scratch_bytes);
int thb200_exchange_fold(void* stream, thb200_exchange* x, int reduce, float* d_out, uint64_t wait_limit_ns);
int thb200_exchange_reduce(void* stream, thb200_exchange* x, int reduce, const thb200_tensor* in, float* d_out,
                           float* scratch, size_t scratch_bytes, uint64_t wait_limit_ns);
int thb200_exchange_destroy(thb200_exchange* x);

/* Bytes of scratch thb200_reduce_dim may need for this shape (0 if none). */
size_t thb200_reduce_dim_scratch_bytes(const thb200_tensor* in, int dim);

/* THClTensor_reduceDim, src/lib/THClReduce.cpp:215-302 with kernels
 * src/lib/THClReduce.cl:30-111: out[..., 0, ...] = fold over `dim`. `out` must
 * already have the shape of `in` with size 1 at `dim`. */
int thb200_reduce_dim(void* stream, int modify, int reduce, const thb200_tensor* out,
                      const thb200_tensor* in, int dim, float init, float mod_param,
                      float* scratch, size_t scratch_bytes);

/* thb200_reduce_dim for hosts that are not allowed to allocate device memory: no
 * counterpart in the reference. Some embedders plan every device buffer up front and
 * forbid allocation afterwards — an inference server with a fixed memory budget, a
 * plugin loaded into another framework's process, a latency-critical loop where
 * cudaMalloc's implicit device synchronisation is unacceptable — so they cannot hand
 * over scratch of their own and the library may not go and get some. Here the scratch
 * is a 4 MiB array inside the library's own device image (held by every GPU that loads
 * the library, until the process exits); the call itself allocates and frees nothing.
 *  - Shapes whose reduction needs more than thb200_reduce_dim_noalloc_capacity() bytes
 *    (see thb200_reduce_dim_scratch_bytes) are refused with an error; use
 *    thb200_reduce_dim with your own scratch for those.
 *  - The first call on each device looks up the array's device address (a one-time
 *    host-side query, done with that device current). Make that first call before
 *    starting any stream capture.
 *  - The array used is the one of the device that is CURRENT when the call is made,
 *    not the device `stream` belongs to: make the stream's device current first, or
 *    the kernel is handed another GPU's array. The cached address does not survive
 *    cudaDeviceReset.
 *  - All calls on a device share the one array and it keeps the previous call's bytes.
 *    Nothing in it has to start at zero (every partial is written before it is read),
 *    but two calls that overlap on the GPU — different streams, or different host
 *    threads without ordering — race on it: keep them on one stream or order them. */
size_t thb200_reduce_dim_noalloc_capacity(void);
int thb200_reduce_dim_noalloc(void* stream, int modify, int reduce, const thb200_tensor* out,
                              const thb200_tensor* in, int dim, float init, float mod_param);

/* THClTensor_reduceDimIndex, src/lib/THClTensorMathTransformReduce.cpp:160-185
 * with kernels src/lib/THClTensorMathTransformReduce.cl:17-102: per slice the
 * extreme value and its 1-based position stored as fp32; strict comparison in
 * ascending position, so the first occurrence wins and NaN never replaces the
 * running value; start value -/+FLT_MAX with index -1. All three tensors are
 * contiguous; src is viewed as [outer][n][inner]. is_max: 1 = max, 0 = min. */
int thb200_reduce_dim_index(void* stream, int is_max, float* values, float* indices, const float* src,
                            int64_t outer, int64_t n, int64_t inner, float* scratch, size_t scratch_bytes);
size_t thb200_reduce_dim_index_scratch_bytes(int64_t outer, int64_t n, int64_t inner);

/* Variance / standard deviation along one dimension in ONE pass over the input:
 * THClTensor_var / THClTensor_std with kernels THClTensor_kernel_varOuterDim /
 * varInnermostDim and THClTensor_computeVar (src/lib/THClTensorMath2.cl:5-108; host side
 * src/lib/THClTensorMath2.cpp:293-333, commented out in the reference and served from there
 * as the specification). biased != 0 divides by n, otherwise by n - 1; negative results of
 * the final subtraction are clamped to 0; apply_sqrt != 0 gives the standard deviation.
 * The sums of (x - k) and (x - k)^2, k = first element of the slice, are kept in double.
 * `out` has the shape of `in` with size 1 at `dim`; any strided layouts. */
size_t thb200_var_dim_scratch_bytes(const thb200_tensor* in, int dim);
int thb200_var_dim(void* stream, const thb200_tensor* out, const thb200_tensor* in, int dim, int biased,
                   int apply_sqrt, float* scratch, size_t scratch_bytes);

/* The same over the whole tensor into *d_out (device pointer): THClTensor_varall /
 * stdall, src/lib/THClTensorMath2.cpp:197-231 (biased = 0 there), in one pass instead of
 * the reference's mean pass followed by a squared-deviation pass. */
size_t thb200_var_all_scratch_bytes(int64_t n);
int thb200_var_all(void* stream, const thb200_tensor* in, int biased, int apply_sqrt, float* d_out,
                   float* scratch, size_t scratch_bytes);

/* Inclusive scan along n of a contiguous tensor viewed as [outer][n][inner]:
 * THClTensor_scanDim with kernels THClTensor_kernel_scanOuterDim / scanInnermostDim
 * (src/lib/THClTensorMathScan.cpp:29-142, src/lib/THClTensorMathScan.cl:27-139); op is
 * THB200_RED_ADD (cumsum, start 0) or THB200_RED_MUL (cumprod, start 1). Running values are
 * kept in double and rounded at each store. dst may be src. When the other dimensions are
 * too small to fill the GPU, n is cut into chunks and `scratch` (8-byte aligned) holds the
 * chunk totals / carries; the pointers matter to the size because 16-byte aligned operands
 * take a different path. Few long rows (inner == 1, n a multiple of 32, 16-byte aligned) are
 * scanned in a single pass by co-resident CTAs (a cooperative launch) that hand each other
 * their tile totals through `scratch`, in a fixed order of additions: results do not vary from
 * run to run. That path and the TMA pipeline over 128-column strips wait on barriers and on
 * words of `scratch`: every such wait is bounded, and a wait that gives up stores a non-zero
 * code into *d_status (a device int the caller keeps at 0 and may read after synchronising;
 * NULL = the library's own word, see thb200_kernel_status) and leaves dst undefined. */
size_t thb200_scan_scratch_bytes(const float* dst, const float* src, int64_t outer, int64_t n, int64_t inner);
int thb200_scan(void* stream, int op, float* dst, const float* src, int64_t outer, int64_t n, int64_t inner,
                void* scratch, size_t scratch_bytes, int* d_status);

/* THClTensor_kernel_renorm, src/lib/THClTensorMath2.cl:110-143 (host side
 * src/lib/THClTensorMath2.cpp:414-446, commented out in the reference): every row of the
 * contiguous [rows][size] matrix whose p-norm exceeds maxnorm is multiplied in place by
 * maxnorm / (norm + 1e-7); other rows are not touched. `scratch` holds one float per row. */
size_t thb200_renorm_rows_scratch_bytes(int64_t rows, int64_t size);
int thb200_renorm_rows(void* stream, float* data, int64_t rows, int64_t size, float p, float maxnorm,
                       void* scratch, size_t scratch_bytes);

/* THClTensor_dist, src/lib/THClTensorMath2.cpp:448-475 (commented out in the reference):
 * *d_out = (sum |a[i] - b[i]|^p)^(1/p) over two contiguous vectors; the sum is kept in
 * double. The result stays on the device. `scratch` must be 8-byte aligned. */
size_t thb200_dist_scratch_bytes(int64_t n);
int thb200_dist(void* stream, const float* a, const float* b, int64_t n, float p, float* d_out, void* scratch,
                size_t scratch_bytes);

/* Fixed-order fold of `count` device floats into *d_out (count <= 1024): the
 * last step of a sum sharded over several GPUs, after the per-GPU partials
 * have been gathered. No counterpart in the reference (it has no collectives). */
int thb200_fold_partials(void* stream, int reduce, const float* d_partials, int count, float* d_out);

/* ---- GEMM ----------------------------------------------------------------- */

/* clblasSgemm as called from THClBlas_gemm, src/lib/THClBlas.cpp:380-449:
 * column-major C(m x n) = alpha * op(A) * op(B) + beta * C, transa/transb 'n' or
 * 't', fp32 in and out. Computed with tcgen05 TF32 tensor-core MMAs on a
 * three-term split of each operand (hi*hi + hi*lo + lo*hi) accumulated in fp32.
 * `batch` independent problems at the given element strides (batch = 1 for addmm).
 * `workspace` holds split operands, split-K partial sums and the status word; size from
 * thb200_gemm_workspace_bytes. How the hi/lo parts reach the tensor core is chosen per problem:
 * long K: A is read in place (either orientation) and split into tensor memory, only B is pre-split;
 * short K / few rows: both operands are read in place and split in shared memory (by pairs of
 * CTAs when there are at least two row tiles); otherwise, and whenever an operand is not 16-byte
 * aligned with a leading dimension that is a multiple of 4, both are pre-split in the workspace.
 * The environment variable THB200_GEMM_MODE = prepass | fused | pair | ts pins the choice where it is
 * eligible (read once per process; for tests and experiments). */
size_t thb200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch);
int thb200_gemm(void* stream, char transa, char transb, int64_t m, int64_t n, int64_t k, float alpha,
                const float* a, int64_t lda, const float* b, int64_t ldb, float beta, float* c, int64_t ldc,
                int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_c,
                void* workspace, size_t workspace_bytes);
/* Every wait inside the GEMM kernel is bounded. Status word of the last
 * thb200_gemm that used this workspace: 0 = completed; 1 = the TMA producer's wait for a free
 * stage, 2 / 6 = the MMA issuer's wait for a loaded / converted stage, 3 = the epilogue's wait for
 * an accumulator, 4 = the MMA issuer's wait for a free accumulator, 5 = a converter's wait for a
 * loaded stage gave up (C is then undefined). Synchronises `stream`.
 * < 0: the status could not be read. */
int thb200_gemm_status(void* stream, int64_t m, int64_t n, int64_t k, int64_t batch, void* workspace);

/* clblasSdot as called from THClBlas_dot, src/lib/THClBlas.cpp:149-192: *d_out =
 * sum a[i] * b[i] over two contiguous vectors; the products are rounded to fp32, their sum
 * is kept in double. The result stays on the device. */
size_t thb200_dot_scratch_bytes(int64_t n);
int thb200_dot(void* stream, const float* a, const float* b, int64_t n, float* d_out, void* scratch,
               size_t scratch_bytes);

/* clblasSgemv as called from THClBlas_gemv, src/lib/THClBlas.cpp:194-262, column-major
 * A (m x n, unit stride along m, leading dimension lda): trans 'n': y(m) = alpha*A*x + beta*y;
 * trans 't': y(n) = alpha*A^T*x + beta*y. HBM-bound: A is read exactly once. */
size_t thb200_gemv_scratch_bytes(char trans, int64_t m, int64_t n);
int thb200_gemv(void* stream, char trans, int64_t m, int64_t n, float alpha, const float* a, int64_t lda,
                const float* x, int64_t incx, float beta, float* y, int64_t incy, void* scratch,
                size_t scratch_bytes);

/* clblasSger as called from THClBlas_ger, src/lib/THClBlas.cpp:264-347: column-major A (m x n,
 * unit stride along m, leading dimension lda): A[i + j*lda] += (alpha * y[j*incy]) * x[i], or
 * (alpha * x[i]) * y[j*incy] when alpha_on_x != 0 (the two differ in the last bit; the THCl layer
 * picks the one that rounds like the reference's operator "*out += val1 * *in1 * *in2").
 * HBM-bound, 8 bytes per element of A. Only the 128-bit path exists: returns 1 and does nothing
 * unless A and x are 16-byte aligned, incx == 1 and m, lda are multiples of 4 (the caller then
 * falls back to the pointwise operator over broadcast views). */
int thb200_ger(void* stream, int64_t m, int64_t n, float alpha, const float* x, int64_t incx, const float* y,
               int64_t incy, float* a, int64_t lda, int alpha_on_x);

/* ---- user kernels ---------------------------------------------------------- */

/* torch.ClKernel, src/UserKernel.cpp:217-381: a kernel whose body the caller writes, with
 * named arguments. A tensor argument `t` appears in the body as `t_info` (pointer to struct
 * THClTensorInfoCl: sizes[25], strides[25], offset, dims; src/lib/THClTensorInfoCl.cl) and
 * `t_data` (start of the storage: the body adds t_info->offset itself), an int or float by
 * its name. The body is compiled by NVRTC as CUDA C++ behind a prelude that defines the
 * OpenCL C words such kernels use (get_global_id(0), get_local_id, get_group_id,
 * get_local_size, get_num_groups, barrier(CLK_LOCAL_MEM_FENCE), global, local, mad);
 * `funcs` is extra source placed before the kernel (functions without a qualifier are
 * device functions). The kernel runs as num_workgroups blocks of workgroup_size threads. */
typedef struct thb200_user_kernel thb200_user_kernel;
enum thb200_arg_kind { THB200_ARG_INT = 0, THB200_ARG_FLOAT = 1, THB200_ARG_TENSOR_IN = 2,
                       THB200_ARG_TENSOR_OUT = 3, THB200_ARG_TENSOR_INOUT = 4 };
typedef struct thb200_user_arg {
  int i;                  /* THB200_ARG_INT */
  float f;                /* THB200_ARG_FLOAT */
  float* storage;         /* tensors: device address of the start of the storage */
  int64_t offset;         /* storage offset of the tensor, in elements */
  int ndim;
  const int64_t* size;
  const int64_t* stride;
} thb200_user_arg;
int thb200_user_kernel_create(const char* name, const char* src, const char* funcs, int nargs,
                              const char* const* arg_names, const int* arg_kinds, thb200_user_kernel** out);
/* The full source that was compiled (ClKernel:getRenderedKernel()). */
const char* thb200_user_kernel_rendered(const thb200_user_kernel* k);
int thb200_user_kernel_run(void* stream, thb200_user_kernel* k, const thb200_user_arg* args, int nargs,
                           int workgroup_size, int64_t num_workgroups);
void thb200_user_kernel_free(thb200_user_kernel* k);

#ifdef __cplusplus
}
#endif
#endif /* THB200_H */
