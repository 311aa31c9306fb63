// Kernel selection and launch for pointwise apply (built-in operators and
// NVRTC-compiled expressions share this path).
#include <cudaTypedefs.h>

#include "thb_internal.h"
#include <unordered_map>
#include "../kernels/math_policy.cuh"
#include "../kernels/apply_kernels.cuh"
#include "../kernels/apply_tma_kernels.cuh"

#include <cstring>

namespace thb {

// Constants of the exact division by d used by thb_fastdiv.
static void fastdiv_constants(uint32_t d, uint32_t* magic, uint32_t* shift) {
  uint32_t l = 0;
  while (l < 32 && (uint64_t(1) << l) < d) ++l;  // ceil(log2 d)
  uint64_t m = ((uint64_t(1) << 32) * ((uint64_t(1) << l) - d)) / d + 1;
  *magic = (uint32_t)m;
  uint32_t sh1 = l < 1 ? l : 1, sh2 = l > 0 ? l - 1 : 0;
  *shift = sh1 | (sh2 << 8);
}

static void fill_layout(ThbLayout* L, float* data, const Collapsed& c) {
  memset(L, 0, sizeof *L);
  L->data = data;
  L->dims = c.dims;
  for (int d = 0; d < c.dims; ++d) {
    L->size[d] = (uint32_t)c.size[d];
    L->stride[d] = (uint32_t)c.stride[d];
    fastdiv_constants((uint32_t)c.size[d], &L->magic[d], &L->shift[d]);
  }
}

// Tensor map of one operand of thb_apply_tile_tma: 32 x 32 boxes with the 128-byte swizzle, the
// unit-stride direction innermost (columns for a row-major operand, rows for a column-major one).
static bool make_tile_map(CUtensorMap* map, const float* data, int64_t inner, int64_t outer, int64_t pitch) {
  auto enc = (PFN_cuTensorMapEncodeTiled_v12000)tensor_map_encoder_ptr();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)pitch * 4};
  cuuint32_t box[2] = {THB_AT_BOX, THB_AT_BOX};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)data, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The TMA tile kernel when the operands qualify: 0 launched, -1 not applicable, 1 error.
// Every apply kernel starts with a grid-dependency wait, so its blocks may be placed while the previous kernel
// of the stream drains (programmatic stream serialisation).
static cudaError_t launch_dependent(const void* func, dim3 grid, dim3 block, void** args, size_t smem, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelExC(&cfg, func, args);
}

static int launch_tile_tma(const ApplyKernels& k, cudaStream_t st, int nt, const ThbTile2d& T, const ThbScalars& s) {
  if (!k.tile_tma || (nt < 2 && !k.reads_out)) return -1;
  const int sms = sm_count();
  const int64_t R = T.R, C = T.C;
  const int64_t tilesC = (C + THB_AT_TILE - 1) / THB_AT_TILE, ntiles = ((R + THB_AT_TILE - 1) / THB_AT_TILE) * tilesC;
  if (R < THB_AT_TILE || C < THB_AT_TILE || ntiles < sms || ntiles > INT32_MAX) return -1;
  CUtensorMap maps[3];
  for (int i = 0; i < nt; ++i) {
    const bool col = (T.colmajor >> i) & 1;
    const int64_t pitch = col ? T.sc[i] : T.sr[i], inner = col ? R : C, outer = col ? C : R;
    if (((uintptr_t)T.data[i] & 15) || (pitch & 3) || pitch < inner || pitch * 4 >= (int64_t(1) << 40)) return -1;
    if (!make_tile_map(&maps[i], T.data[i], inner, outer, pitch)) return -1;
  }
  for (int i = nt; i < 3; ++i) maps[i] = maps[0];
  ThbTileTma P;
  P.R = (uint32_t)R; P.C = (uint32_t)C; P.tilesC = (uint32_t)tilesC; P.ntiles = (uint32_t)ntiles;
  P.colmajor = T.colmajor; P.status = device_status_word(STATUS_TILE_APPLY);
  P.tilesR = (uint32_t)((R + THB_AT_TILE - 1) / THB_AT_TILE);
  P.band = 8;  // measured on 8192 x 8192: 0.91-0.95 of the copy rate with bands of 4-8 tile rows, 0.84-0.90 row by row
  const size_t smem = THB_AT_SMEM(nt);
  if (cudaFuncSetAttribute(k.tile_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();  // not launchable with this much shared memory here: the thread-staged kernel takes over
    return -1;
  }
  ThbScalars sc = s;
  void* args[] = {&maps[0], &maps[1], &maps[2], &P, &sc};
  THB_CUDA(launch_dependent(k.tile_tma, dim3((unsigned)(ntiles < sms ? ntiles : sms)), dim3(THB_AT_THREADS), args, smem, st));
  return 0;
}

static int misalign_elems(const float* p) {  // elements before the next 16-byte boundary
  return (int)(((16 - ((uintptr_t)p & 15)) & 15) >> 2);
}

int launch_apply(const ApplyKernels& k, cudaStream_t st, int nt, const thb200_tensor* t, float val1,
                 float val2, const float* p1, const float* p2, bool dry_run, int* plan_out) {
  if (plan_out) *plan_out = PLAN_NONE;
  if (nt < 1 || nt > 3) return fail("apply: %d tensors (1..3 supported)", nt);
  if (k.nt != nt) return fail("apply: operator %s takes %d tensors, got %d", k.name ? k.name : "?", k.nt, nt);
  for (int i = 0; i < nt; ++i)
    if (t[i].ndim > THB200_MAX_DIMS) return fail("Apply: too many dimensions in tensor %d", i + 1);
  const int64_t n = num_elements(t[0]);
  for (int i = 1; i < nt; ++i)
    if (num_elements(t[i]) != n) return fail("element size mismatch between tensors 1 and %d", i + 1);
  if (n == 0) return 0;
  for (int i = 0; i < nt; ++i)
    if (!t[i].data) return fail("apply: tensor %d has no device memory", i + 1);

  Collapsed c[3];
  bool all_contig = true;
  for (int i = 0; i < nt; ++i) {
    if (!collapse(t[i].ndim, t[i].size, t[i].stride, -1, &c[i])) return fail("apply: bad layout in tensor %d", i + 1);
    all_contig = all_contig && c[i].contiguous();
  }
  ThbScalars s{val1, val2, p1, p2};

  if (all_contig) {
    int head = misalign_elems(t[0].data);
    bool same_phase = ((uintptr_t)t[0].data & 3) == 0;
    for (int i = 1; i < nt; ++i) same_phase = same_phase && misalign_elems(t[i].data) == head;
    if (same_phase) {
      if (plan_out) *plan_out = PLAN_CONTIG;
      if (dry_run) return 0;
      if (head > n) head = (int)n;
      float* a = t[0].data;
      const float* b = nt >= 2 ? t[1].data : nullptr;
      const float* cc = nt >= 3 ? t[2].data : nullptr;
      int64_t nn = n;
      int64_t nvec = (n - head) >> 2;
      int64_t blocks = (nvec + THB_CONTIG_THREADS * THB_CONTIG_UNROLL - 1) / (THB_CONTIG_THREADS * THB_CONTIG_UNROLL);
      int64_t cap = kMaxGridBlocks;
      if (blocks > cap) blocks = cap;
      if (blocks < 1) blocks = 1;
      // start at the end that the previous streaming kernel left in L2 (bit 8 of the head argument)
      const void* ptrs[3] = {a, b, cc};
      const bool descending = stream_prefers_descending(ptrs, nt, (size_t)n * sizeof(float));
      stream_note_end(ptrs, nt, (size_t)n * sizeof(float), descending);
      if (descending) head |= 256;
      void* args[] = {&a, &b, &cc, &nn, &head, &s};
      THB_CUDA(launch_dependent(k.contig, dim3((unsigned)blocks), dim3(THB_CONTIG_THREADS), args, 0, st));
      return 0;
    }
  }

  for (int i = 0; i < nt; ++i)
    if (!can_use_32bit(t[i].ndim, t[i].size, t[i].stride))
      return fail("apply: tensor %d needs 64-bit index math on a non-contiguous layout: not implemented", i + 1);

  // 2-D paths: every operand is the same R x C matrix (a contiguous one counts as R x C).
  {
    int64_t R = 0, C = 0;
    bool ok = true, any_col = false;
    for (int i = 0; i < nt && ok; ++i)
      if (c[i].dims == 2) {
        if (R == 0) { R = c[i].size[0]; C = c[i].size[1]; }
        else if (R != c[i].size[0] || C != c[i].size[1]) ok = false;
      } else if (c[i].dims != 1) ok = false;
    // rows path: unit stride along C everywhere, float4 along the rows
    if (ok && R > 0 && R * C == n && (C & 3) == 0 && k.rows2d) {
      ThbRows2d Q;
      memset(&Q, 0, sizeof Q);
      bool rows_ok = true;
      for (int i = 0; i < nt && rows_ok; ++i) {
        Q.data[i] = t[i].data;
        if (c[i].dims == 1) {
          rows_ok = c[i].stride[0] == 1;
          Q.row_stride[i] = C;
        } else {
          rows_ok = c[i].stride[1] == 1 && (c[i].stride[0] & 3) == 0;
          Q.row_stride[i] = c[i].stride[0];
        }
        rows_ok = rows_ok && ((uintptr_t)t[i].data & 15) == 0;
      }
      const uint64_t nvec = (uint64_t)R * (uint64_t)(C >> 2);
      if (rows_ok && nvec < (uint64_t(1) << 32)) {
        if (plan_out) *plan_out = PLAN_ROWS2D;
        if (dry_run) return 0;
        Q.cvec = (uint32_t)(C >> 2);
        fastdiv_constants(Q.cvec, &Q.magic, &Q.shift);
        Q.nvec = nvec;
        uint64_t per_block = THB_CONTIG_THREADS * THB_CONTIG_UNROLL;
        uint64_t blocks = (nvec + per_block - 1) / per_block;
        uint64_t cap = (uint64_t)kMaxGridBlocks;
        if (blocks > cap) blocks = cap;
        void* args[] = {&Q, &s};
        THB_CUDA(launch_dependent(k.rows2d, dim3((unsigned)blocks), dim3(THB_CONTIG_THREADS), args, 0, st));
        return 0;
      }
    }
    // tile path: at least one operand is column-major-like
    if (ok && R > 0 && R * C == n && k.tile2d) {
      ThbTile2d P;
      memset(&P, 0, sizeof P);
      for (int i = 0; i < nt && ok; ++i) {
        P.data[i] = t[i].data;
        if (c[i].dims == 1) {
          if (c[i].stride[0] != 1) ok = false;
          P.sr[i] = C; P.sc[i] = 1;
        } else {
          P.sr[i] = c[i].stride[0]; P.sc[i] = c[i].stride[1];
          if (P.sc[i] == 1) {}
          else if (P.sr[i] == 1) { P.colmajor |= 1 << i; any_col = true; }
          else ok = false;
        }
      }
      if (ok && any_col) {
        if (plan_out) *plan_out = PLAN_TILE2D;
        if (dry_run) return 0;
        P.R = (uint32_t)R; P.C = (uint32_t)C;
        // large matrices: tiles move through the TMA unit
        if (const int rc = launch_tile_tma(k, st, nt, P, s); rc >= 0) return rc;
        // 128-bit variant when every access it makes is 16-byte aligned
        bool v4 = k.tile2d_v4 != nullptr;
        for (int i = 0; i < nt && v4; ++i) {
          v4 = ((uintptr_t)t[i].data & 15) == 0;
          if ((P.colmajor >> i) & 1) v4 = v4 && (R & 3) == 0 && (P.sc[i] & 3) == 0;
          else v4 = v4 && (C & 3) == 0 && (P.sr[i] & 3) == 0;
        }
        if (v4) {
          P.tilesC = (uint32_t)((C + THB_T4_C - 1) / THB_T4_C);
          uint64_t ntiles = (uint64_t)((R + THB_T4_R - 1) / THB_T4_R) * P.tilesC;
          P.ntiles = (uint32_t)ntiles;
          uint64_t blocks = ntiles;
          uint64_t cap = (uint64_t)kMaxGridBlocks;
          if (blocks > cap) blocks = cap;
          void* args[] = {&P, &s};
          THB_CUDA(launch_dependent(k.tile2d_v4, dim3((unsigned)blocks), dim3(256), args, 0, st));
          return 0;
        }
        P.tilesC = (uint32_t)((C + THB_TILE - 1) / THB_TILE);
        uint64_t ntiles = (uint64_t)((R + THB_TILE - 1) / THB_TILE) * P.tilesC;
        P.ntiles = (uint32_t)ntiles;
        uint64_t blocks = ntiles;
        uint64_t cap = (uint64_t)kMaxGridBlocks;
        if (blocks > cap) blocks = cap;
        void* args[] = {&P, &s};
        THB_CUDA(launch_dependent(k.tile2d, dim3((unsigned)blocks), dim3(THB_TILE, THB_TILE_ROWS), args, 0, st));
        return 0;
      }
    }
  }

  if (plan_out) *plan_out = PLAN_STRIDED;
  if (dry_run) return 0;
  ThbLayout L[3];
  memset(L, 0, sizeof L);
  for (int i = 0; i < nt; ++i) fill_layout(&L[i], t[i].data, c[i]);
  uint64_t nn = (uint64_t)n;
  uint64_t per_block = THB_STRIDED_THREADS * THB_STRIDED_UNROLL;
  uint64_t blocks = (nn + per_block - 1) / per_block;
  uint64_t cap = (uint64_t)kMaxGridBlocks;
  if (blocks > cap) blocks = cap;
  void* args[] = {&L[0], &L[1], &L[2], &nn, &s};
  THB_CUDA(launch_dependent(k.strided, dim3((unsigned)blocks), dim3(THB_STRIDED_THREADS), args, 0, st));
  return 0;
}

}  // namespace thb

extern "C" {

int thb200_op_code(const char* name) {
  if (!name) return -1;
  // name -> code, built on the first call (the operator table is constant)
  static const std::unordered_map<std::string, int>* table = [] {
    auto* m = new std::unordered_map<std::string, int>();
    for (int i = 0; i < thb::builtin_op_count(); ++i) m->emplace(thb::builtin_op(i)->name, i);
    return m;
  }();
  auto it = table->find(name);
  return it == table->end() ? -1 : it->second;
}

int thb200_op_arity(int op) {
  const thb::ApplyKernels* k = thb::builtin_op(op);
  return k ? k->nt : -1;
}

int thb200_apply_plan(int ntensors, const thb200_tensor* t) {
  thb::ApplyKernels k;
  k.nt = ntensors;
  k.tile2d = (const void*)1;  // eligibility only; nothing is launched
  k.rows2d = (const void*)1;
  int plan = 0;
  if (thb::launch_apply(k, nullptr, ntensors, t, 0, 0, nullptr, nullptr, true, &plan)) return -1;
  return plan;
}

int thb200_apply_op(void* stream, int op, int ntensors, const thb200_tensor* t, float val1, float val2,
                    const float* point1, const float* point2) {
  THB_TIMED(stream, "thb200_apply_op");
  const thb::ApplyKernels* k = thb::builtin_op(op);
  if (!k) return thb::fail("apply: unknown operator code %d", op);
  return thb::launch_apply(*k, (cudaStream_t)stream, ntensors, t, val1, val2, point1, point2, false, nullptr);
}

int thb200_apply_expr(void* stream, const char* body, int ntensors, const thb200_tensor* t, float val1,
                      float val2, const float* point1, const float* point2) {
  THB_TIMED(stream, "thb200_apply_expr");
  if (!body) return thb::fail("apply: null expression");
  const thb::ApplyKernels* k = nullptr;
  if (int rc = thb::expr_kernels(ntensors, body, &k)) return rc;
  return thb::launch_apply(*k, (cudaStream_t)stream, ntensors, t, val1, val2, point1, point2, false, nullptr);
}

}  // extern "C"
