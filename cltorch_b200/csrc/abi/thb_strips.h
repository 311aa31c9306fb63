// Host-side planning of the TMA strip pipeline (kernels/reduce_strip_kernels.cuh), shared by
// the reductions and the matrix-vector product.
#pragma once
#include <cudaTypedefs.h>

#include "thb_internal.h"

namespace thb {

struct StripPlan {
  bool ok = false;
  int strips_per_outer = 0, total_strips = 0;
  uint32_t nchunks = 1, chunk_rows = 0;
};

// Whether a reduction over n of a contiguous [outer][n][inner] tensor should go through the strip
// pipeline, and into how many row chunks: the fewest (up to 16) that fill the SMs to 97 %
// over whole rounds of work items; without enough items the one-thread-per-column path stays.
static inline StripPlan plan_strips(const float* src, int64_t outer, int64_t n, int64_t inner) {
  StripPlan p;
  if (((uintptr_t)src & 15) != 0 || (inner & 3) != 0 || inner < 4 || n < 256) return p;
  if (inner >= (int64_t(1) << 31) || outer >= (int64_t(1) << 31) || n >= (int64_t(1) << 31) ||
      n * inner * 4 >= (int64_t(1) << 40) || outer * inner >= (int64_t(1) << 32))
    return p;
  if (!tensor_map_encoder_ptr()) return p;
  const int64_t spo = (inner + THB_SS_COLS - 1) / THB_SS_COLS, total = spo * outer;
  if (total >= (int64_t(1) << 24)) return p;
  const int sms = sm_count();
  const int64_t max_c = n / 256 < 16 ? n / 256 : 16;
  int64_t best_c = 1;
  double best_eff = 0.0;
  for (int64_t c = 1; c <= max_c; ++c) {
    const int64_t items = total * c, rounds = (items + sms - 1) / sms;
    const double eff = (double)items / (double)(rounds * sms);
    if (eff > best_eff + 1e-9) { best_eff = eff; best_c = c; }
    if (eff >= 0.97) break;
  }
  if (best_eff < 0.8) return p;
  int64_t rows = (n + best_c - 1) / best_c;
  rows = (rows + THB_SS_ROWS - 1) / THB_SS_ROWS * THB_SS_ROWS;
  p.chunk_rows = (uint32_t)rows;
  p.nchunks = (uint32_t)((n + rows - 1) / rows);
  p.strips_per_outer = (int)spo;
  p.total_strips = (int)total;
  p.ok = true;
  return p;
}

// Tensor map over [outer][n][inner] floats whose rows are `pitch` elements apart (pitch a multiple of 4).
static inline int make_strip_map(CUtensorMap* map, const float* src, int64_t outer, int64_t n, int64_t inner,
                                 int64_t pitch) {
  auto enc = (PFN_cuTensorMapEncodeTiled_v12000)tensor_map_encoder_ptr();
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)n, (cuuint64_t)outer};
  cuuint64_t strides[2] = {(cuuint64_t)pitch * 4, (cuuint64_t)pitch * 4 * (cuuint64_t)n};
  cuuint32_t box[3] = {THB_SS_COLS, THB_SS_ROWS, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)src, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("reduce: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}


}  // namespace thb
