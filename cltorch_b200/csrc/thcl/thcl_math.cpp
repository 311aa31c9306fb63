// Front-ends of the pointwise, reduction and BLAS functions of include/THCl.h:
// argument checks, resizing, operator choice and overlap handling as in the
// reference's src/lib/THClTensorMath*.cpp; the arithmetic is in the CUDA
// kernels behind include/thb200.h.
#include "thcl_internal.h"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>

using namespace thcl;

namespace thcl {

static void same_device(THClState* state, int n, THClTensor** t) {
  for (int i = 1; i < n; ++i)
    if (t[i] && t[0] && t[i]->device != t[0]->device) raise("tensors are on different devices");
  (void)state;
}

void pointwise(THClState* state, int nt, THClTensor** tensors, const bool* read_write, const char* op, const char* expr,
               float val1, float val2, const THClTensor* point1) {
  same_device(state, nt, tensors);
  const long n = THClTensor_nElement(state, tensors[0]);
  for (int t = 1; t < nt; ++t)
    if (THClTensor_nElement(state, tensors[t]) != n) raise("element size mismatch between tensors 1 and %d", t + 1);
  for (int t = 0; t < nt; ++t)
    if (tensors[t]->nDimension > THB200_MAX_DIMS) raise("tensor too large or too many (>%d) dimensions", THB200_MAX_DIMS);
  if (n == 0) return;
  const int device = tensors[0]->device;
  THClDeviceContext* ctx = context(state, device);
  use_device(device);

  // A read/write operand whose indices overlap goes through a contiguous copy
  // and is copied back, last writer wins (reference src/lib/THClApply.cpp:174-190,231-237).
  THClTensor* original[3] = {nullptr, nullptr, nullptr};
  for (int t = 0; t < nt; ++t) {
    if (read_write[t]) {
      View v;
      v.set(tensors[t]);
      if (thb200_overlapping_indices(v.t.ndim, v.size, v.stride)) {
        original[t] = tensors[t];
        tensors[t] = THClTensor_newContiguous(state, tensors[t]);
      }
    }
  }

  const float* p1 = nullptr;
  if (point1) {
    if (!point1->storage || !point1->storage->wrapper) raise("point tensor has no storage");
    p1 = point1->storage->wrapper + point1->storageOffset;
  }
  View v[3];
  thb200_tensor tt[3];
  for (int t = 0; t < nt; ++t) {
    v[t].set(tensors[t]);
    tt[t] = v[t].t;
  }
  int rc;
  if (op) {
    int code = thb200_op_code(op);
    if (code < 0) raise("unknown built-in operator %s", op);
    rc = thb200_apply_op(ctx->stream, code, nt, tt, val1, val2, p1, nullptr);
  } else {
    rc = thb200_apply_expr(ctx->stream, expr, nt, tt, val1, val2, p1, nullptr);
  }
  std::string err = rc ? thb200_last_error() : "";
  for (int t = 0; t < nt; ++t) {
    if (original[t]) {
      if (!rc) THClTensor_copyIgnoringOverlaps(state, original[t], tensors[t]);
      THClTensor_free(state, tensors[t]);
      tensors[t] = original[t];
    }
  }
  if (rc) raise("%s", err.c_str());
  after_launch(state, ctx);
}

static void apply1(THClState* state, THClTensor* a, const char* op, float v1 = 0.f, float v2 = 0.f,
                   const THClTensor* pt = nullptr) {
  THClTensor* t[1] = {a};
  const bool rw[1] = {true};
  pointwise(state, 1, t, rw, op, nullptr, v1, v2, pt);
}
static void apply2(THClState* state, THClTensor* a, THClTensor* b, const char* op, float v1 = 0.f, float v2 = 0.f,
                   const THClTensor* pt = nullptr, bool a_rw = true) {
  THClTensor* t[2] = {a, b};
  const bool rw[2] = {a_rw, false};
  pointwise(state, 2, t, rw, op, nullptr, v1, v2, pt);
}
static void apply3(THClState* state, THClTensor* a, THClTensor* b, THClTensor* c, const char* op, float v1 = 0.f,
                   float v2 = 0.f) {
  THClTensor* t[3] = {a, b, c};
  const bool rw[3] = {true, false, false};
  pointwise(state, 3, t, rw, op, nullptr, v1, v2, nullptr);
}

// self = f(src): in place when self == src, else resize self like src and use
// the two-tensor form (the pattern of IMPLEMENT_CL_TENSOR_BASIC_FUNC,
// reference src/lib/THClTensorMathPointwise.cpp:18-37).
static void unary_like(THClState* state, THClTensor* self, THClTensor* src, const char* op1, const char* op2,
                       float v1 = 0.f, float v2 = 0.f, const THClTensor* pt = nullptr) {
  if (self == src) {
    apply1(state, self, op1, v1, v2, pt);
  } else {
    THClTensor_resizeAs(state, self, src);
    apply2(state, self, src, op2, v1, v2, pt);
  }
}

// self = src1 OP src2: two-tensor form when self == src1.
static void binary_like(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2, const char* op2,
                        const char* op3, float v1 = 0.f) {
  arg_check(THClTensor_nElement(state, src1) == THClTensor_nElement(state, src2), 3, "sizes do not match");
  if (self == src1) {
    apply2(state, self, src2, op2, v1);
  } else {
    THClTensor_resizeAs(state, self, src1);
    apply3(state, self, src1, src2, op3, v1);
  }
}

static void check_point(const THClTensor* value) {
  arg_check(value->nDimension == 0, 4, "must be a point tensor (zero dimensions)");
  arg_check(value->storage != nullptr, 4, "point tensor must have allocated storage");
}

// ---- reductions -------------------------------------------------------------

static void reduce_all(THClState* state, THClTensor* src, int mod, int red, float init, float mparam,
                       const float* mpoint, int fin, float fparam, float* d_out) {
  if (src->nDimension > THB200_MAX_DIMS) raise("tensor too large or too many (>%d) dimensions", THB200_MAX_DIMS);
  THClDeviceContext* ctx = context(state, src->device);
  use_device(src->device);
  View v;
  v.set(src);
  const long n = THClTensor_nElement(state, src);
  size_t need = thb200_reduce_all_scratch_bytes(n);
  float* scratch = ensure_scratch(ctx, need);
  check_thb(thb200_reduce_all(ctx->stream, mod, red, &v.t, init, mparam, mpoint, fin, fparam, d_out, scratch,
                              ctx->scratch_bytes));
  after_launch(state, ctx);
}

// Reads back result slot `slot` of the device's result buffer: the blocking step
// of the host-scalar reductions (scratch->wrapper->copyToHost() in the reference).
static float read_result(THClState* state, THClDeviceContext* ctx, int slot) {
  if (state->trace) printf("THCl: device -> host 1 float (reduction result)\n");
  return read_host_result(ctx, slot);
}

static float reduce_all_host(THClState* state, THClTensor* self, int mod, int red, float init, float mparam = 0.f) {
  THClDeviceContext* ctx = context(state, self->device);
  reduce_all(state, self, mod, red, init, mparam, nullptr, THB200_FIN_NONE, 1.f, host_result_target(ctx));
  return read_result(state, ctx, 0);
}

static void reduce_all_point(THClState* state, THClTensor* self, THClTensor* src, int mod, int red, float init) {
  if (self->device != src->device) raise("tensors are on different devices");
  THClTensor_resize0d(state, self);
  reduce_all(state, src, mod, red, init, 0.f, nullptr, THB200_FIN_NONE, 1.f, self->storage->wrapper + self->storageOffset);
}

static void moments_point(THClState* state, THClTensor* src, int what /*0 mean, 1 var, 2 std*/, float* d_out) {
  arg_check(src->nDimension > 0, 1, "empty Tensor");
  THClDeviceContext* ctx = context(state, src->device);
  const long n = THClTensor_nElement(state, src);
  if (what == 0) {
    reduce_all(state, src, THB200_MOD_COPY, THB200_RED_ADD, 0.f, 0.f, nullptr, THB200_FIN_DIV, (float)n, d_out);
    return;
  }
  // one pass over the input (shifted sums of x and x^2 in double) instead of the reference's
  // mean pass followed by a squared-deviation pass (src/lib/THClTensorMath2.cpp:209-229)
  if (src->nDimension > THB200_MAX_DIMS) raise("tensor too large or too many (>%d) dimensions", THB200_MAX_DIMS);
  use_device(src->device);
  View v;
  v.set(src);
  float* scratch = ensure_scratch(ctx, thb200_var_all_scratch_bytes(n));
  check_thb(thb200_var_all(ctx->stream, &v.t, 0, what == 2, d_out, scratch, ctx->scratch_bytes));
  after_launch(state, ctx);
}

static void reduce_dim(THClState* state, THClTensor* self, THClTensor* src, int mod, int red, float init, float mparam,
                       long dim) {
  if (self->device != src->device) raise("tensors are on different devices");
  if (src->nDimension > THB200_MAX_DIMS) raise("tensor too large or too many (>%d) dimensions", THB200_MAX_DIMS);
  if (src->nDimension <= 0) return;  // zero-dim tensor: nothing to do (reference src/lib/THClReduce.cpp:233-236)
  arg_check(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  THLongStorage* sizes = THClTensor_newSizeOf(state, src);
  sizes->data[dim] = 1;
  THClTensor_resize(state, self, sizes, nullptr);
  THLongStorage_free(sizes);
  THClDeviceContext* ctx = context(state, src->device);
  use_device(src->device);
  View vo, vi;
  vo.set(self);
  vi.set(src);
  size_t need = thb200_reduce_dim_scratch_bytes(&vi.t, (int)dim);
  float* scratch = ensure_scratch(ctx, need);
  check_thb(thb200_reduce_dim(ctx->stream, mod, red, &vo.t, &vi.t, (int)dim, init, mparam, scratch, ctx->scratch_bytes));
  after_launch(state, ctx);
}

static void reduce_dim_index(THClState* state, THClTensor* values_, THClTensor* indices_, THClTensor* src, long dim,
                             int is_max) {
  arg_check(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  if (values_->device != src->device || indices_->device != src->device) raise("tensors are on different devices");
  THLongStorage* sizes = THClTensor_newSizeOf(state, src);
  sizes->data[dim] = 1;
  THClTensor_resize(state, values_, sizes, nullptr);
  THClTensor_resize(state, indices_, sizes, nullptr);
  THLongStorage_free(sizes);
  // The reference makes contiguous copies of all three (src/lib/THClTensorMathTransformReduce.cpp:172-174).
  // The copy of the source is skipped for the transposed view of a contiguous matrix: reducing it
  // along one dimension is reducing the matrix underneath along the other, positions along the
  // reduced dimension and the order of the results are the same, so the kernels run on the
  // storage as it lies (a transposed 1 GiB input would otherwise pay 8 bytes per element for the
  // copy before a 4-byte-per-element reduction).
  THClTensor* values = THClTensor_newContiguous(state, values_);
  THClTensor* indices = THClTensor_newContiguous(state, indices_);
  const bool transposed2d = src->nDimension == 2 && src->size[0] > 1 && src->size[1] > 1 && src->stride[0] == 1 &&
                            src->stride[1] == src->size[0];
  THClTensor* in = transposed2d ? src : THClTensor_newContiguous(state, src);
  int64_t outer = 1, inner = 1, n = 0;
  if (transposed2d) {
    // underneath: a contiguous size[1] x size[0] matrix; dimension `dim` of the view is dimension 1 - dim there
    n = src->size[dim];
    if (dim == 0) outer = src->size[1];   // innermost dimension of the matrix underneath
    else inner = src->size[0];            // its outer dimension
  } else {
    for (int d = 0; d < dim; ++d) outer *= in->size[d];
    for (int d = (int)dim + 1; d < in->nDimension; ++d) inner *= in->size[d];
    n = in->size[dim];
  }
  THClDeviceContext* ctx = context(state, src->device);
  use_device(src->device);
  size_t need = thb200_reduce_dim_index_scratch_bytes(outer, n, inner);
  float* scratch = ensure_scratch(ctx, need);
  int rc = thb200_reduce_dim_index(ctx->stream, is_max, THClTensor_data(state, values), THClTensor_data(state, indices),
                                   THClTensor_data(state, in), outer, n, inner, scratch, ctx->scratch_bytes);
  std::string err = rc ? thb200_last_error() : "";
  if (!transposed2d) THClTensor_free(state, in);
  THClTensor_freeCopyTo(state, values, values_);
  THClTensor_freeCopyTo(state, indices, indices_);
  if (rc) raise("%s", err.c_str());
  after_launch(state, ctx);
}

}  // namespace thcl

extern "C" {

// ---- fills -------------------------------------------------------------------

void THClTensor_fill(THClState* state, THClTensor* self, float value) {
  THCL_BEGIN
  apply1(state, self, "FILL_1", value);
  THCL_END_VOID
}
void THClTensor_zero(THClState* state, THClTensor* self) { THClTensor_fill(state, self, 0.f); }
void THClTensor_zeros(THClState* state, THClTensor* r_, THLongStorage* size) {
  THCL_BEGIN
  THClTensor_resize(state, r_, size, nullptr);
  THClTensor_zero(state, r_);
  THCL_END_VOID
}
void THClTensor_ones(THClState* state, THClTensor* r_, THLongStorage* size) {
  THCL_BEGIN
  THClTensor_resize(state, r_, size, nullptr);
  THClTensor_fill(state, r_, 1.f);
  THCL_END_VOID
}
void THClTensor_reshape(THClState* state, THClTensor* r_, THClTensor* t, THLongStorage* size) {
  THCL_BEGIN
  THClTensor_resize(state, r_, size, nullptr);
  THClTensor_copy(state, r_, t);
  THCL_END_VOID
}
long THClTensor_numel(THClState* state, THClTensor* t) { return THClTensor_nElement(state, t); }

void THClTensor_fill_gpu(THClState* state, THClTensor* self, THClTensor* value) {
  THCL_BEGIN
  check_point(value);
  apply1(state, self, "FILLPT_1", 0.f, 0.f, value);
  THCL_END_VOID
}

// ---- scalar and point-tensor arithmetic (src/lib/THClTensorMathPairwise.cpp) ---

void THClTensor_add(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  unary_like(state, self, src, "ADDC_1", "ADDC_2", value);
  THCL_END_VOID
}
void THClTensor_sub(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  unary_like(state, self, src, "ADDC_1", "ADDC_2", -value);
  THCL_END_VOID
}
void THClTensor_mul(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  unary_like(state, self, src, "MULC_1", "MULC_2", value);
  THCL_END_VOID
}
void THClTensor_div(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  arg_check(value != 0.0f, 3, "divide by zero");
  unary_like(state, self, src, "MULC_1", "MULC_2", 1.0f / value);
  THCL_END_VOID
}
void THClTensor_add_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value) {
  THCL_BEGIN
  check_point(value);
  unary_like(state, self, src, "ADDPT_1", "ADDPT_2", 0.f, 0.f, value);
  THCL_END_VOID
}
void THClTensor_sub_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value) {
  THCL_BEGIN
  check_point(value);
  unary_like(state, self, src, "SUBPT_1", "SUBPT_2", 0.f, 0.f, value);
  THCL_END_VOID
}
void THClTensor_mul_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value) {
  THCL_BEGIN
  check_point(value);
  unary_like(state, self, src, "MULPT_1", "MULPT_2", 0.f, 0.f, value);
  THCL_END_VOID
}
void THClTensor_div_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value) {
  THCL_BEGIN
  check_point(value);
  unary_like(state, self, src, "DIVPT_1", "DIVPT_2", 0.f, 0.f, value);
  THCL_END_VOID
}

// ---- tensor-tensor arithmetic -------------------------------------------------

void THClTensor_cadd(THClState* state, THClTensor* self, THClTensor* src1, float value, THClTensor* src2) {
  THCL_BEGIN
  if (src2->nDimension == 0) {  // a point tensor on the right (src/lib/THClTensorMathPointwise.cpp:151-154)
    THClTensor_add_gpu(state, self, src1, src2);
    return;
  }
  if (value == 1.0f) binary_like(state, self, src1, src2, "ADD_2", "ADD_3");
  else binary_like(state, self, src1, src2, "CADD_2", "CADD_3", value);
  THCL_END_VOID
}
void THClTensor_csub(THClState* state, THClTensor* self, THClTensor* src1, float value, THClTensor* src2) {
  THCL_BEGIN
  if (src2->nDimension == 0) {
    THClTensor_sub_gpu(state, self, src1, src2);
    return;
  }
  if (value == 1.0f) binary_like(state, self, src1, src2, "SUB_2", "SUB_3");
  else binary_like(state, self, src1, src2, "CSUB_2", "CSUB_3", value);
  THCL_END_VOID
}
void THClTensor_cmul(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2) {
  THCL_BEGIN
  binary_like(state, self, src1, src2, "MUL_2", "MUL_3");
  THCL_END_VOID
}
void THClTensor_cdiv(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2) {
  THCL_BEGIN
  binary_like(state, self, src1, src2, "DIV_2", "DIV_3");
  THCL_END_VOID
}
void THClTensor_cpow(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2) {
  THCL_BEGIN
  binary_like(state, self, src1, src2, "CPOW_2", "CPOW_3");
  THCL_END_VOID
}
void THClTensor_cmax(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2) {
  THCL_BEGIN
  binary_like(state, self, src1, src2, "CMAX_2", "CMAX_3");
  THCL_END_VOID
}
void THClTensor_cmin(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2) {
  THCL_BEGIN
  binary_like(state, self, src1, src2, "CMIN_2", "CMIN_3");
  THCL_END_VOID
}
void THClTensor_cmaxValue(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  unary_like(state, self, src, "CMAXV_1", "CMAXV_2", value);
  THCL_END_VOID
}
void THClTensor_cminValue(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  unary_like(state, self, src, "CMINV_1", "CMINV_2", value);
  THCL_END_VOID
}

// self = t + value * src1 * src2: t is first copied into self when they differ
// (src/lib/THClTensorMath.cpp:194-216)
static void addc(THClState* state, THClTensor* self, THClTensor* t, float value, THClTensor* src1, THClTensor* src2,
                 const char* op) {
  if (self != t) {
    THClTensor_resizeAs(state, self, t);
    THClTensor_copy(state, self, t);
  } else {
    arg_check(THClTensor_nElement(state, self) == THClTensor_nElement(state, src1), 1, "sizes do not match");
  }
  arg_check(THClTensor_nElement(state, src1) == THClTensor_nElement(state, src2), 3, "sizes do not match");
  apply3(state, self, src1, src2, op, value);
}
void THClTensor_addcmul(THClState* state, THClTensor* self, THClTensor* t, float value, THClTensor* src1, THClTensor* src2) {
  THCL_BEGIN
  addc(state, self, t, value, src1, src2, "ADDCMUL_3");
  THCL_END_VOID
}
void THClTensor_addcdiv(THClState* state, THClTensor* self, THClTensor* t, float value, THClTensor* src1, THClTensor* src2) {
  THCL_BEGIN
  addc(state, self, t, value, src1, src2, "ADDCDIV_3");
  THCL_END_VOID
}

// ---- unary functions ------------------------------------------------------------

#define THCL_UNARY(NAME, OP)                                                        \
  void THClTensor_##NAME(THClState* state, THClTensor* self, THClTensor* src) {     \
    THCL_BEGIN                                                                      \
    unary_like(state, self, src, #OP "_1", #OP "_2");                               \
    THCL_END_VOID                                                                   \
  }
THCL_UNARY(log, LOG) THCL_UNARY(log1p, LOG1P) THCL_UNARY(exp, EXP) THCL_UNARY(cos, COS)
THCL_UNARY(acos, ACOS) THCL_UNARY(cosh, COSH) THCL_UNARY(sin, SIN) THCL_UNARY(asin, ASIN)
THCL_UNARY(sinh, SINH) THCL_UNARY(tan, TAN) THCL_UNARY(atan, ATAN) THCL_UNARY(tanh, TANH)
THCL_UNARY(sqrt, SQRT) THCL_UNARY(ceil, CEIL) THCL_UNARY(floor, FLOOR) THCL_UNARY(abs, ABS)
THCL_UNARY(round, ROUND) THCL_UNARY(neg, NEG) THCL_UNARY(cinv, CINV) THCL_UNARY(sigmoid, SIGMOID)
THCL_UNARY(sign, SIGN)
#undef THCL_UNARY

void THClTensor_pow(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  // integer-valued exponent: pown, defined for negative bases (src/lib/THClTensorMath2.cpp:22-44)
  const bool integral = (float)(int)value == value;
  unary_like(state, self, src, integral ? "POWN_1" : "POW_1", integral ? "POWN_2" : "POW_2", value);
  THCL_END_VOID
}
void THClTensor_tpow(THClState* state, THClTensor* self, float value, THClTensor* src) {
  THCL_BEGIN
  unary_like(state, self, src, "TPOW_1", "TPOW_2", value);
  THCL_END_VOID
}
void THClTensor_clamp(THClState* state, THClTensor* self, THClTensor* src, float min_value, float max_value) {
  THCL_BEGIN
  unary_like(state, self, src, "CLAMP_1", "CLAMP_2", min_value, max_value);
  THCL_END_VOID
}
void THClTensor_atan2(THClState* state, THClTensor* r_, THClTensor* tx, THClTensor* ty) {
  THCL_BEGIN
  arg_check(THClTensor_nElement(state, tx) == THClTensor_nElement(state, ty), 3, "sizes do not match");
  THClTensor_resizeAs(state, r_, tx);
  apply3(state, r_, tx, ty, "ATAN2_3");
  THCL_END_VOID
}

// ---- comparisons ------------------------------------------------------------------

#define THCL_COMPARE(NAME, OP)                                                                                   \
  void THClTensor_##NAME##Value(THClState* state, THClTensor* self_, THClTensor* src, float value) {             \
    THCL_BEGIN                                                                                                   \
    THClTensor_resizeAs(state, self_, src);                                                                      \
    apply2(state, self_, src, #OP "V_2", value);                                                                 \
    THCL_END_VOID                                                                                                \
  }                                                                                                              \
  void THClTensor_##NAME##PointTensor(THClState* state, THClTensor* self_, THClTensor* src, THClTensor* value) { \
    THCL_BEGIN                                                                                                   \
    check_point(value);                                                                                          \
    THClTensor_resizeAs(state, self_, src);                                                                      \
    apply2(state, self_, src, #OP "PT_2", 0.f, 0.f, value);                                                      \
    THCL_END_VOID                                                                                                \
  }                                                                                                              \
  void THClTensor_##NAME##Tensor(THClState* state, THClTensor* self_, THClTensor* src1, THClTensor* src2) {      \
    THCL_BEGIN                                                                                                   \
    if (src2->nDimension == 0) {                                                                                 \
      THClTensor_##NAME##PointTensor(state, self_, src1, src2);                                                  \
      return;                                                                                                    \
    }                                                                                                            \
    THClTensor_resizeAs(state, self_, src1);                                                                     \
    arg_check(THClTensor_nElement(state, src1) == THClTensor_nElement(state, src2), 3, "sizes do not match");    \
    apply3(state, self_, src1, src2, #OP "T_3");                                                                 \
    THCL_END_VOID                                                                                                \
  }
THCL_COMPARE(lt, LT) THCL_COMPARE(gt, GT) THCL_COMPARE(le, LE)
THCL_COMPARE(ge, GE) THCL_COMPARE(eq, EQ) THCL_COMPARE(ne, NE)
#undef THCL_COMPARE

// ---- user expressions ---------------------------------------------------------------

static void user_expr(THClState* state, int nt, THClTensor** t, const char* expression) {
  arg_check(expression != nullptr, nt + 1, "expression expected");
  std::string out(strlen(expression) * 8 + 64, '\0');
  int n = thb200_rewrite_expr(expression, nt, &out[0], out.size());
  if (n < 0) raise("expression too long");
  out.resize(n);
  const bool rw[3] = {true, false, false};
  pointwise(state, nt, t, rw, nullptr, out.c_str(), 0.f, 0.f, nullptr);
}
void THClTensor_apply(THClState* state, THClTensor* self, char const* operation1) {
  THCL_BEGIN
  THClTensor* t[1] = {self};
  user_expr(state, 1, t, operation1);
  THCL_END_VOID
}
void THClTensor_map(THClState* state, THClTensor* self, THClTensor* two, char const* operation2) {
  THCL_BEGIN
  THClTensor* t[2] = {self, two};
  user_expr(state, 2, t, operation2);
  THCL_END_VOID
}
void THClTensor_map2(THClState* state, THClTensor* self, THClTensor* in1, THClTensor* in2, char const* operation3) {
  THCL_BEGIN
  THClTensor* t[3] = {self, in1, in2};
  user_expr(state, 3, t, operation3);
  THCL_END_VOID
}

// ---- whole-tensor reductions (src/lib/THClTensorMath.cpp:259-528) ---------------------

float THClTensor_sumall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  return reduce_all_host(state, self, THB200_MOD_COPY, THB200_RED_ADD, 0.f);
  THCL_END(0.f)
}
float THClTensor_prodall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  return reduce_all_host(state, self, THB200_MOD_COPY, THB200_RED_MUL, 1.f);
  THCL_END(0.f)
}
float THClTensor_minall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  return reduce_all_host(state, self, THB200_MOD_COPY, THB200_RED_MIN, INFINITY);
  THCL_END(0.f)
}
float THClTensor_maxall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  return reduce_all_host(state, self, THB200_MOD_COPY, THB200_RED_MAX, -INFINITY);
  THCL_END(0.f)
}
int THClTensor_logicalall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  return (int)reduce_all_host(state, self, THB200_MOD_COPY, THB200_RED_AND, 1.f);
  THCL_END(0)
}
int THClTensor_logicalany(THClState* state, THClTensor* self) {
  THCL_BEGIN
  return (int)reduce_all_host(state, self, THB200_MOD_COPY, THB200_RED_OR, 0.f);
  THCL_END(0)
}
float THClTensor_meanall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  arg_check(self->nDimension > 0, 1, "empty Tensor");
  return THClTensor_sumall(state, self) / THClTensor_nElement(state, self);
  THCL_END(0.f)
}
float THClTensor_varall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  THClDeviceContext* ctx = context(state, self->device);
  moments_point(state, self, 1, host_result_target(ctx));
  return read_result(state, ctx, 0);
  THCL_END(0.f)
}
float THClTensor_stdall(THClState* state, THClTensor* self) {
  THCL_BEGIN
  THClDeviceContext* ctx = context(state, self->device);
  moments_point(state, self, 2, host_result_target(ctx));
  return read_result(state, ctx, 0);
  THCL_END(0.f)
}
float THClTensor_normall(THClState* state, THClTensor* self, float value) {
  THCL_BEGIN
  if (value == 0.0f) return reduce_all_host(state, self, THB200_MOD_NEZERO, THB200_RED_ADD, 0.f);
  float r = reduce_all_host(state, self, THB200_MOD_ABSPOW, THB200_RED_ADD, 0.f, value);
  return powf(r, 1.0f / value);
  THCL_END(0.f)
}
float THClTensor_as_float(THClState* state, THClTensor* self) {
  THCL_BEGIN
  arg_check(self->nDimension == 0, 1, "tensor must be point tensor, zero dimensions");
  arg_check(self->storage != nullptr, 1, "tensor must have allocated storage");
  return THClStorage_get(state, self->storage, self->storageOffset);
  THCL_END(0.f)
}

void THClTensor_sumall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  reduce_all_point(state, self, src, THB200_MOD_COPY, THB200_RED_ADD, 0.f);
  THCL_END_VOID
}
void THClTensor_prodall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  reduce_all_point(state, self, src, THB200_MOD_COPY, THB200_RED_MUL, 1.f);
  THCL_END_VOID
}
void THClTensor_minall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  reduce_all_point(state, self, src, THB200_MOD_COPY, THB200_RED_MIN, INFINITY);
  THCL_END_VOID
}
void THClTensor_maxall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  reduce_all_point(state, self, src, THB200_MOD_COPY, THB200_RED_MAX, -INFINITY);
  THCL_END_VOID
}
void THClTensor_logicalall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  reduce_all_point(state, self, src, THB200_MOD_COPY, THB200_RED_AND, 1.f);
  THCL_END_VOID
}
void THClTensor_logicalany_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  reduce_all_point(state, self, src, THB200_MOD_COPY, THB200_RED_OR, 0.f);
  THCL_END_VOID
}
static void moments_gpu(THClState* state, THClTensor* self, THClTensor* src, int what) {
  if (self->device != src->device) raise("tensors are on different devices");
  THClTensor_resize0d(state, self);
  moments_point(state, src, what, self->storage->wrapper + self->storageOffset);
}
void THClTensor_meanall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  moments_gpu(state, self, src, 0);
  THCL_END_VOID
}
void THClTensor_varall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  moments_gpu(state, self, src, 1);
  THCL_END_VOID
}
void THClTensor_stdall_gpu(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  moments_gpu(state, self, src, 2);
  THCL_END_VOID
}

// ---- reductions along one dimension ---------------------------------------------------

void THClTensor_sum(THClState* state, THClTensor* self, THClTensor* src, long dim) {
  THCL_BEGIN
  reduce_dim(state, self, src, THB200_MOD_COPY, THB200_RED_ADD, 0.f, 0.f, dim);
  THCL_END_VOID
}
void THClTensor_prod(THClState* state, THClTensor* self, THClTensor* src, long dim) {
  THCL_BEGIN
  reduce_dim(state, self, src, THB200_MOD_COPY, THB200_RED_MUL, 1.f, 0.f, dim);
  THCL_END_VOID
}
void THClTensor_mean(THClState* state, THClTensor* self, THClTensor* src, long dim) {
  THCL_BEGIN
  // sum, then the scalar div, i.e. a multiplication by 1/size (src/lib/THClTensorMath2.cpp:188-194)
  THClTensor_sum(state, self, src, dim);
  THClTensor_div(state, self, self, (float)THClTensor_size(state, src, (int)dim));
  THCL_END_VOID
}
void THClTensor_norm(THClState* state, THClTensor* self, THClTensor* src, float value, long dimension) {
  THCL_BEGIN
  if (value == 0.0f) {
    reduce_dim(state, self, src, THB200_MOD_NEZERO, THB200_RED_ADD, 0.f, 0.f, dimension);
  } else {
    reduce_dim(state, self, src, THB200_MOD_ABSPOW, THB200_RED_ADD, 0.f, value, dimension);
    THClTensor_pow(state, self, self, 1 / value);
  }
  THCL_END_VOID
}
void THClTensor_max(THClState* state, THClTensor* values, THClTensor* indices, THClTensor* src, long dim) {
  THCL_BEGIN
  reduce_dim_index(state, values, indices, src, dim, 1);
  THCL_END_VOID
}
void THClTensor_min(THClState* state, THClTensor* values, THClTensor* indices, THClTensor* src, long dim) {
  THCL_BEGIN
  reduce_dim_index(state, values, indices, src, dim, 0);
  THCL_END_VOID
}

}  // extern "C"

// ---- variance / standard deviation along one dimension, scans, renorm, dist ---------------

static void var_dim(THClState* state, THClTensor* self, THClTensor* src, long dim, int flag, int apply_sqrt) {
  if (self->device != src->device) raise("tensors are on different devices");
  if (src->nDimension > THB200_MAX_DIMS) raise("tensor too large or too many (>%d) dimensions", THB200_MAX_DIMS);
  arg_check(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  // the result keeps the dimension with size 1 (src/lib/THClTensorMath2.cpp:296-299)
  THLongStorage* sizes = THClTensor_newSizeOf(state, src);
  sizes->data[dim] = 1;
  THClTensor_resize(state, self, sizes, nullptr);
  THLongStorage_free(sizes);
  THClDeviceContext* ctx = context(state, src->device);
  use_device(src->device);
  View vo, vi;
  vo.set(self);
  vi.set(src);
  float* scratch = ensure_scratch(ctx, thb200_var_dim_scratch_bytes(&vi.t, (int)dim));
  check_thb(thb200_var_dim(ctx->stream, &vo.t, &vi.t, (int)dim, flag, apply_sqrt, scratch, ctx->scratch_bytes));
  after_launch(state, ctx);
}

static void scan_dim(THClState* state, THClTensor* self_, THClTensor* src, long dim, int op) {
  if (self_->device != src->device) raise("tensors are on different devices");
  arg_check(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  // THClTensor_scanDim, src/lib/THClTensorMathScan.cpp:127-142: resize, contiguous copies of both
  THClTensor_resizeAs(state, self_, src);
  THClTensor* self = THClTensor_newContiguous(state, self_);
  THClTensor* in = THClTensor_newContiguous(state, src);
  int64_t outer = 1, inner = 1;
  for (int d = 0; d < dim; ++d) outer *= in->size[d];
  for (int d = (int)dim + 1; d < in->nDimension; ++d) inner *= in->size[d];
  const int64_t n = in->size[dim];
  THClDeviceContext* ctx = context(state, src->device);
  use_device(src->device);
  float* dst = THClTensor_data(state, self);
  const float* sp = THClTensor_data(state, in);
  void* scratch = ensure_scratch(ctx, thb200_scan_scratch_bytes(dst, sp, outer, n, inner));
  int rc = thb200_scan(ctx->stream, op, dst, sp, outer, n, inner, scratch, ctx->scratch_bytes, nullptr);
  std::string err = rc ? thb200_last_error() : "";
  THClTensor_free(state, in);
  THClTensor_freeCopyTo(state, self, self_);
  if (rc) raise("%s", err.c_str());
  after_launch(state, ctx);
}

extern "C" {

void THClTensor_var(THClState* state, THClTensor* self, THClTensor* src, long dimension, int flag) {
  THCL_BEGIN
  var_dim(state, self, src, dimension, flag, 0);
  THCL_END_VOID
}
void THClTensor_std(THClState* state, THClTensor* self, THClTensor* src, long dimension, int flag) {
  THCL_BEGIN
  var_dim(state, self, src, dimension, flag, 1);
  THCL_END_VOID
}
void THClTensor_cumsum(THClState* state, THClTensor* self, THClTensor* src, long dimension) {
  THCL_BEGIN
  scan_dim(state, self, src, dimension, THB200_RED_ADD);
  THCL_END_VOID
}
void THClTensor_cumprod(THClState* state, THClTensor* self, THClTensor* src, long dimension) {
  THCL_BEGIN
  scan_dim(state, self, src, dimension, THB200_RED_MUL);
  THCL_END_VOID
}

void THClTensor_renorm(THClState* state, THClTensor* self, THClTensor* src, float value, long dimension, float maxnorm) {
  THCL_BEGIN
  if (self->device != src->device) raise("tensors are on different devices");
  arg_check(dimension >= 0 && dimension < THClTensor_nDimension(state, src), 3, "invalid dimension");
  arg_check(value > 0, 2, "non-positive-norm not supported");
  arg_check(THClTensor_nDimension(state, src) > 1, 1, "need at least 2 dimensions");
  THClDeviceContext* ctx = context(state, src->device);
  use_device(src->device);
  // src/lib/THClTensorMath2.cpp:414-446: the sub-tensors along `dimension` become the rows of a
  // contiguous clone of the transposed source, are rescaled in place, and the clone is copied
  // back transposed. In place on a contiguous tensor along dimension 0 the clone is not needed.
  const bool direct = self == src && dimension == 0 && THClTensor_isContiguous(state, src);
  THClTensor* data = nullptr;
  if (direct) {
    data = self;
  } else {
    THClTensor* src_t = THClTensor_newTranspose(state, src, (int)dimension, 0);
    data = THClTensor_newClone(state, src_t);
    THClTensor_free(state, src_t);
  }
  const int64_t rows = data->size[0];
  const int64_t size = rows > 0 ? THClTensor_nElement(state, data) / rows : 0;
  void* scratch = ensure_scratch(ctx, thb200_renorm_rows_scratch_bytes(rows, size));
  int rc = thb200_renorm_rows(ctx->stream, THClTensor_data(state, data), rows, size, value, maxnorm, scratch,
                              ctx->scratch_bytes);
  std::string err = rc ? thb200_last_error() : "";
  if (!direct) {
    if (!rc) {
      THClTensor* back = THClTensor_newTranspose(state, data, (int)dimension, 0);
      THClTensor_resizeAs(state, self, back);
      THClTensor_copy(state, self, back);
      THClTensor_free(state, back);
    }
    THClTensor_free(state, data);
  }
  if (rc) raise("%s", err.c_str());
  after_launch(state, ctx);
  THCL_END_VOID
}

// Both tensors have the same sizes and strides, and those strides are a permutation of a contiguous
// layout: the elements fill [data, data + nElement) without gaps, in the same order in both.
static bool same_dense_layout(const THClTensor* a, const THClTensor* b) {
  if (a->nDimension != b->nDimension || a->nDimension < 1 || a->nDimension > 8) return false;
  int order[8], nd = 0;
  for (int d = 0; d < a->nDimension; ++d) {
    if (a->size[d] != b->size[d] || a->stride[d] != b->stride[d]) return false;
    if (a->size[d] == 0) return false;
    if (a->size[d] > 1) order[nd++] = d;
  }
  for (int i = 1; i < nd; ++i)           // by ascending stride
    for (int j = i; j > 0 && a->stride[order[j]] < a->stride[order[j - 1]]; --j) { int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t; }
  long expect = 1;
  for (int i = 0; i < nd; ++i) {
    if (a->stride[order[i]] != expect) return false;
    expect *= a->size[order[i]];
  }
  return true;
}

static void dist_into(THClState* state, THClTensor* self, THClTensor* src, float value, float* d_out) {
  if (self->device != src->device) raise("tensors are on different devices");
  arg_check(THClTensor_nElement(state, self) == THClTensor_nElement(state, src), 2, "sizes do not match");
  THClDeviceContext* ctx = context(state, self->device);
  use_device(self->device);
  // contiguous copies of both, as src/lib/THClTensorMath2.cpp:463-465 - unless the two tensors lie in
  // memory in the same way and without gaps (e.g. both transposed): the distance is a sum over pairs of
  // elements, and walking both storages front to back pairs the same elements
  const bool same_dense = same_dense_layout(self, src);
  THClTensor* a = same_dense ? self : THClTensor_newContiguous(state, self);
  THClTensor* b = same_dense ? src : THClTensor_newContiguous(state, src);
  const long n = THClTensor_nElement(state, self);
  void* scratch = ensure_scratch(ctx, thb200_dist_scratch_bytes(n));
  int rc = thb200_dist(ctx->stream, THClTensor_data(state, a), THClTensor_data(state, b), n, value, d_out, scratch,
                       ctx->scratch_bytes);
  std::string err = rc ? thb200_last_error() : "";
  if (!same_dense) {
    THClTensor_free(state, a);
    THClTensor_free(state, b);
  }
  if (rc) raise("%s", err.c_str());
  after_launch(state, ctx);
}

float THClTensor_dist(THClState* state, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  THClDeviceContext* ctx = context(state, self->device);
  dist_into(state, self, src, value, host_result_target(ctx));
  return read_result(state, ctx, 0);
  THCL_END(0.f)
}
// The distance as a point tensor: no host synchronisation.
void THClTensor_dist_gpu(THClState* state, THClTensor* res, THClTensor* self, THClTensor* src, float value) {
  THCL_BEGIN
  if (res->device != self->device) raise("tensors are on different devices");
  THClTensor_resize0d(state, res);
  dist_into(state, self, src, value, res->storage->wrapper + res->storageOffset);
  THCL_END_VOID
}

}  // extern "C"
