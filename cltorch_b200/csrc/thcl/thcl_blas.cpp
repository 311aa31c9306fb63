// addmm and baddbmm: operand normalisation for a column-major GEMM, as
// THClTensor_addmm does it (reference src/lib/THClTensorMathBlas.cpp:107-214),
// then thb200_gemm. baddbmm is declared but not implemented in the reference
// (src/lib/THClTensorMathBlas.cpp:279-428 ends in THError("Not implemented"));
// it follows the same rules per batch: r_b = beta * t_b + alpha * a_b * b_b.
#include "thcl_internal.h"

using namespace thcl;

namespace {

struct Operand {
  THClTensor* t;     // tensor actually passed to the GEMM (may be a contiguous copy)
  THClTensor* owned; // non-null when `t` must be freed
  char trans;
  long ld;
};

// One matrix operand of a column-major GEMM whose result is laid out with unit
// stride along dimension `d0` (d1 = the other one): usable as is when either of
// its two strides is 1, otherwise through a contiguous copy.
Operand normalise(THClState* state, THClTensor* m, int d0, int d1, int base) {
  Operand o{m, nullptr, 'n', 0};
  if (m->stride[base + d0] == 1 && m->stride[base + d1] >= (m->size[base + d0] > 1 ? m->size[base + d0] : 1)) {
    o.trans = 'n';
    o.ld = m->stride[base + d1];
  } else if (m->stride[base + d1] == 1 && m->stride[base + d0] >= (m->size[base + d1] > 1 ? m->size[base + d1] : 1)) {
    o.trans = 't';
    o.ld = m->stride[base + d0];
  } else {
    o.owned = THClTensor_newContiguous(state, m);
    o.t = o.owned;
    // a contiguous (row-major) matrix has unit stride along its last dimension
    o.trans = (d0 == 0 ? 't' : 'n');
    o.ld = o.t->stride[base];
  }
  long min_ld = (o.trans == 'n') ? m->size[base + d0] : m->size[base + d1];
  if (o.ld < min_ld) o.ld = min_ld;
  if (o.ld < 1) o.ld = 1;
  return o;
}

void gemm_front(THClState* state, THClTensor* r_, float beta, THClTensor* t, float alpha, THClTensor* m1, THClTensor* m2,
                bool batched) {
  const int base = batched ? 1 : 0;
  const int nd = batched ? 3 : 2;
  if (m1->nDimension != nd || m2->nDimension != nd)
    raise(batched ? "expected 3D tensors (batch x rows x cols)" : "matrix and matrix expected");
  if (t->nDimension != nd) raise("size mismatch");
  if (t->size[base] != m1->size[base] || t->size[base + 1] != m2->size[base + 1] || m1->size[base + 1] != m2->size[base])
    raise("size mismatch");
  if (batched && (t->size[0] != m1->size[0] || t->size[0] != m2->size[0])) raise("equal number of batches expected");
  if (r_->device != t->device || m1->device != t->device || m2->device != t->device) raise("tensors are on different devices");

  if (t != r_) {
    THClTensor_resizeAs(state, r_, t);
    THClTensor_copy(state, r_, t);
  }

  // result: column-major when stride[0] == 1; row-major (stride[1] == 1) is the
  // column-major transpose, computed as r^T = m2^T m1^T by swapping the operands
  THClTensor* r = r_;
  THClTensor* r_owned = nullptr;
  bool swapped = false;
  const long rows = r_->size[base], cols = r_->size[base + 1];
  if (r_->stride[base] == 1 && r_->stride[base + 1] >= (rows > 1 ? rows : 1)) {
    swapped = false;
  } else if (r_->stride[base + 1] == 1 && r_->stride[base] >= (cols > 1 ? cols : 1)) {
    swapped = true;
  } else {
    r_owned = THClTensor_newContiguous(state, r_);  // row-major copy, written back at the end
    r = r_owned;
    swapped = true;
  }
  THClTensor* a = swapped ? m2 : m1;
  THClTensor* b = swapped ? m1 : m2;
  const int d0 = swapped ? 1 : 0, d1 = swapped ? 0 : 1;
  Operand oa = normalise(state, a, d0, d1, base);
  Operand ob = normalise(state, b, d0, d1, base);

  const long m = r->size[base + d0], n = r->size[base + d1], k = a->size[base + d1];
  long ldc = r->stride[base + d1];
  if (ldc < (m > 1 ? m : 1)) ldc = (m > 1 ? m : 1);
  const long batch = batched ? r->size[0] : 1;

  THClDeviceContext* ctx = context(state, r->device);
  use_device(r->device);
  size_t ws_bytes = thb200_gemm_workspace_bytes(m, n, k, batch);
  void* ws = ensure_gemm_ws(ctx, ws_bytes);
  int rc = thb200_gemm(ctx->stream, oa.trans, ob.trans, m, n, k, alpha, THClTensor_data(state, oa.t), oa.ld,
                       THClTensor_data(state, ob.t), ob.ld, beta, THClTensor_data(state, r), ldc, batch,
                       batched ? oa.t->stride[0] : 0, batched ? ob.t->stride[0] : 0, batched ? r->stride[0] : 0, ws,
                       ctx->gemm_ws_bytes);
  if (!rc) {
    ctx->gemm_pending = true;
    ctx->gemm_shape[0] = m; ctx->gemm_shape[1] = n; ctx->gemm_shape[2] = k; ctx->gemm_shape[3] = batch;
  }
  std::string err = rc ? thb200_last_error() : "";
  if (oa.owned) THClTensor_free(state, oa.owned);
  if (ob.owned) THClTensor_free(state, ob.owned);
  if (r_owned) THClTensor_freeCopyTo(state, r_owned, r_);
  if (rc) raise("%s", err.c_str());
  after_launch(state, ctx);
}

}  // namespace

extern "C" {

void THClTensor_addmm(THClState* state, THClTensor* r_, float beta, THClTensor* t, float alpha, THClTensor* m1, THClTensor* m2) {
  THCL_BEGIN
  gemm_front(state, r_, beta, t, alpha, m1, m2, false);
  THCL_END_VOID
}

void THClTensor_baddbmm(THClState* state, THClTensor* result, float beta, THClTensor* t, float alpha, THClTensor* batch1, THClTensor* batch2) {
  THCL_BEGIN
  gemm_front(state, result, beta, t, alpha, batch1, batch2, true);
  THCL_END_VOID
}

float THClTensor_dot(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  arg_check(THClTensor_nElement(state, self) == THClTensor_nElement(state, src), 2, "sizes do not match");
  if (self->device != src->device) raise("tensors are on different devices");
  // contiguous copies of strided operands, as the reference does
  THClTensor* a = THClTensor_newContiguous(state, self);
  THClTensor* b = THClTensor_newContiguous(state, src);
  THClDeviceContext* ctx = context(state, self->device);
  use_device(self->device);
  const long n = THClTensor_nElement(state, a);
  float* scratch = ensure_scratch(ctx, thb200_dot_scratch_bytes(n));
  int rc = thb200_dot(ctx->stream, THClTensor_data(state, a), THClTensor_data(state, b), n, host_result_target(ctx), scratch,
                      ctx->scratch_bytes);
  std::string err = rc ? thb200_last_error() : "";
  THClTensor_free(state, a);
  THClTensor_free(state, b);
  if (rc) raise("%s", err.c_str());
  return read_host_result(ctx, 0);
  THCL_END(0.f)
}

void THClTensor_addmv(THClState* state, THClTensor* r_, float beta, THClTensor* t, float alpha, THClTensor* mat, THClTensor* vec) {
  THCL_BEGIN
  if (mat->nDimension != 2 || vec->nDimension != 1) raise("matrix and vector expected");
  if (mat->size[1] != vec->size[0]) raise("size mismatch");
  if (t->nDimension != 1) raise("size mismatch");
  if (t->size[0] != mat->size[0]) raise("size mismatch");
  if (r_->device != t->device || mat->device != t->device || vec->device != t->device) raise("tensors are on different devices");
  if (r_ != t) {
    THClTensor_resizeAs(state, r_, t);
    THClTensor_copy(state, r_, t);
  }
  // a matrix with unit stride along its rows index is the column-major 'n' case;
  // a row-major one is its transpose; anything else goes through a contiguous copy
  THClTensor* owned = nullptr;
  char trans;
  long m, n, lda;
  if (mat->stride[0] == 1 && mat->stride[1] >= (mat->size[0] > 1 ? mat->size[0] : 1)) {
    trans = 'n'; m = mat->size[0]; n = mat->size[1]; lda = mat->stride[1];
  } else {
    if (!(mat->stride[1] == 1 && mat->stride[0] >= (mat->size[1] > 1 ? mat->size[1] : 1))) {
      owned = THClTensor_newContiguous(state, mat);
      mat = owned;
    }
    trans = 't'; m = mat->size[1]; n = mat->size[0]; lda = mat->stride[0];
    if (lda < (m > 1 ? m : 1)) lda = (m > 1 ? m : 1);
  }
  THClDeviceContext* ctx = context(state, r_->device);
  use_device(r_->device);
  float* scratch = ensure_scratch(ctx, thb200_gemv_scratch_bytes(trans, m, n));
  int rc = thb200_gemv(ctx->stream, trans, m, n, alpha, THClTensor_data(state, mat), lda, THClTensor_data(state, vec),
                       vec->stride[0], beta, THClTensor_data(state, r_), r_->stride[0], scratch, ctx->scratch_bytes);
  std::string err = rc ? thb200_last_error() : "";
  if (owned) THClTensor_free(state, owned);
  if (rc) raise("%s", err.c_str());
  after_launch(state, ctx);
  THCL_END_VOID
}

void THClTensor_addr(THClState* state, THClTensor* r_, float beta, THClTensor* t, float alpha, THClTensor* vec1, THClTensor* vec2) {
  THCL_BEGIN
  if (vec1->nDimension != 1 || vec2->nDimension != 1) raise("vector and vector expected");
  if (t->nDimension != 2) raise("size mismatch");
  if (t->size[0] != vec1->size[0] || t->size[1] != vec2->size[0]) raise("size mismatch");
  if (r_ != t) {
    THClTensor_resizeAs(state, r_, t);
    THClTensor_copy(state, r_, t);
  }
  if (beta != 1) THClTensor_mul(state, r_, r_, beta);
  // The rank-1 update r += alpha * vec1 (x) vec2. A result with unit-stride rows or columns takes
  // the 128-bit kernel behind thb200_ger (same rounding order as the operator below) ...
  if (r_->storage && vec1->storage && vec2->storage && THClTensor_nElement(state, r_) > 0) {
    THClDeviceContext* ctx = context(state, r_->device);
    use_device(r_->device);
    float* rp = THClTensor_data(state, r_);
    const float* p1 = THClTensor_data(state, vec1);
    const float* p2 = THClTensor_data(state, vec2);
    int rc = 1;
    if (r_->stride[1] == 1 && vec2->stride[0] == 1)        // rows contiguous: the unit-stride index is vec2's
      rc = thb200_ger(ctx->stream, r_->size[1], r_->size[0], alpha, p2, 1, p1, vec1->stride[0], rp, r_->stride[0], 0);
    else if (r_->stride[0] == 1 && vec1->stride[0] == 1)   // columns contiguous (a transposed result)
      rc = thb200_ger(ctx->stream, r_->size[0], r_->size[1], alpha, p1, 1, p2, vec2->stride[0], rp, r_->stride[1], 1);
    if (rc == 0) { after_launch(state, ctx); return; }
    if (rc != 1) raise("%s", thb200_last_error());
  }
  // ... any other layout the pointwise operator
  // "*out += val1 * *in1 * *in2" over broadcast (stride-0) views of the two vectors
  THClTensor* a = THClTensor_newWithStorage2d(state, vec1->device, vec1->storage, vec1->storageOffset, vec1->size[0],
                                              vec1->stride[0], vec2->size[0], 0);
  THClTensor* b = THClTensor_newWithStorage2d(state, vec2->device, vec2->storage, vec2->storageOffset, vec1->size[0], 0,
                                              vec2->size[0], vec2->stride[0]);
  try {
    THClTensor* ts[3] = {r_, a, b};
    const bool rw[3] = {true, false, false};
    pointwise(state, 3, ts, rw, "ADDCMUL_3", nullptr, alpha, 0.f, nullptr);
  } catch (...) {
    THClTensor_free(state, a);
    THClTensor_free(state, b);
    throw;
  }
  THClTensor_free(state, a);
  THClTensor_free(state, b);
  THCL_END_VOID
}

}  // extern "C"
