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

}  // extern "C"
