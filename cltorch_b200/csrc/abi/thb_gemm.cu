// Host side of thb200_gemm: operand split, TMA descriptors, launch.
#include "thb_internal.h"
#include "../kernels/gemm_ts_kernels.cuh"
#include "../kernels/gemm_pair_kernels.cuh"

#include <cudaTypedefs.h>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace thb {

static int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// cuTensorMapEncodeTiled through the runtime, so that the library does not link libcuda.
void* tensor_map_encoder_ptr();
static PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() { return (PFN_cuTensorMapEncodeTiled_v12000)tensor_map_encoder_ptr(); }
void* tensor_map_encoder_ptr() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  });
  return (void*)fn;
}

static const int kKPad = 32;  // K is padded to this in the split operands (a multiple of every BK)

// [parts = 2 * batch][rows][Kp] fp32, box bk x box_rows x 1, swizzle span = one box row.
static int make_operand_map(CUtensorMap* map, const float* base, int64_t rows, int64_t Kp, int64_t parts, int box_rows,
                            int bk) {
  auto enc = tensor_map_encoder();
  if (!enc) return fail("gemm: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)Kp, (cuuint64_t)rows, (cuuint64_t)parts};
  cuuint64_t strides[2] = {(cuuint64_t)Kp * 4, (cuuint64_t)Kp * 4 * (cuuint64_t)rows};
  cuuint32_t box[3] = {(cuuint32_t)bk, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("gemm: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

// The caller's own matrix as a TMA tensor: element (row r, k) at base[r * sr + k * sk] with one of the
// two strides equal to 1. K-major (sk == 1): dimensions (k, rows, batch), box bk x box_rows x 1 with the
// swizzle span of one box row; MN-major (sr == 1): dimensions (rows, k, batch), box 32 x bk x 1 with the
// 128-byte swizzle in 32-byte atoms (the only layout the tensor core transposes 32-bit operands from). Out-of-range parts of a box read as zero, which is what pads K and the edge tiles.
static int make_raw_operand_map(CUtensorMap* map, const float* base, bool mn_major, int64_t rows, int64_t k, int64_t ld,
                                int64_t batch, int64_t batch_stride, int box_rows, int bk) {
  auto enc = tensor_map_encoder();
  if (!enc) return fail("gemm: cuTensorMapEncodeTiled is not available from this driver");
  const int64_t inner = mn_major ? rows : k, outer = mn_major ? k : rows;
  const int64_t bstride = batch > 1 ? batch_stride : ld * outer;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)bstride * 4};
  cuuint32_t box[3] = {(cuuint32_t)(mn_major ? 32 : bk), (cuuint32_t)(mn_major ? bk : box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                         : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("gemm: cuTensorMapEncodeTiled failed with %d on a caller matrix", (int)r);
  return 0;
}

// A' for the tensor-memory kernel: MN-major caller matrix as (rows, k, batch), box 128 x bk x 1, no swizzle
// (the converter warps read it with one thread per row).
static int make_raw_rows_map(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int64_t batch,
                             int64_t batch_stride, int bk) {
  auto enc = tensor_map_encoder();
  if (!enc) return fail("gemm: cuTensorMapEncodeTiled is not available from this driver");
  const int64_t bstride = batch > 1 ? batch_stride : ld * k;
  cuuint64_t dims[3] = {(cuuint64_t)rows, (cuuint64_t)k, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)bstride * 4};
  cuuint32_t box[3] = {THB_GEMM_BM, (cuuint32_t)bk, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("gemm: cuTensorMapEncodeTiled failed with %d on a caller matrix", (int)r);
  return 0;
}

// Whether TMA can read this operand in place: 16-byte aligned base, leading dimension and batch
// stride multiples of 4 floats, extents within the tensor-map limits.
static bool raw_operand_ok(const float* base, int64_t ld, int64_t batch, int64_t batch_stride) {
  if (((uintptr_t)base & 15) != 0 || (ld & 3) != 0 || ld <= 0) return false;
  if (batch > 1 && ((batch_stride & 3) != 0 || batch_stride <= 0)) return false;
  if ((uint64_t)ld * 4 >= (1ull << 40) || (batch > 1 && (uint64_t)batch_stride * 4 >= (1ull << 40))) return false;
  return true;
}

struct Workspace {
  float* a;  // [batch][2][m][Kp]
  float* b;  // [batch][2][n][Kp]
  float* partial;  // [splits][batch][n][m], only for problems that may be split along K
  int* status;
  size_t bytes;
};

// Split-K is considered for problems with at most this many 128 x 256 tiles (a constant, so
// that the workspace size does not depend on the device), with up to kMaxSplits splits.
static const int64_t kSplitTileLimit = 96;
static const int kMaxSplits = 4;
static int64_t tiles256_of(int64_t m, int64_t n, int64_t batch) {
  return ((m + THB_GEMM_BM - 1) / THB_GEMM_BM) * ((n + 255) / 256) * batch;
}

static Workspace carve(void* ws, int64_t m, int64_t n, int64_t k, int64_t batch) {
  const int64_t Kp = round_up(k, kKPad);
  Workspace w;
  ws = (void*)(((uintptr_t)ws + 1023) & ~(uintptr_t)1023);  // TMA and the swizzle want 1024-byte aligned bases
  size_t a_bytes = (size_t)round_up(batch * 2 * m * Kp * 4, 1024);
  size_t b_bytes = (size_t)round_up(batch * 2 * n * Kp * 4, 1024);
  w.a = (float*)ws;
  w.b = (float*)((char*)ws + a_bytes);
  size_t p_bytes = 0;
  if (tiles256_of(m, n, batch) <= kSplitTileLimit && Kp >= 1024)
    p_bytes = (size_t)round_up((int64_t)kMaxSplits * batch * m * n * 4, 1024);
  w.partial = (float*)((char*)ws + a_bytes + b_bytes);
  w.status = (int*)((char*)ws + a_bytes + b_bytes + p_bytes);
  w.bytes = a_bytes + b_bytes + p_bytes + 1024 /*status*/ + 1024 /*alignment slack*/;
  return w;
}

}  // namespace thb

using namespace thb;

extern "C" {

size_t thb200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch) {
  if (m <= 0 || n <= 0 || k <= 0 || batch <= 0) return 1024;
  return carve(nullptr, m, n, k, batch).bytes;
}

int thb200_gemm(void* stream, char transa, char transb, int64_t m, int64_t n, int64_t k, float alpha, const float* a,
                int64_t lda, const float* b, int64_t ldb, float beta, float* c, int64_t ldc, int64_t batch,
                int64_t stride_a, int64_t stride_b, int64_t stride_c, void* workspace, size_t workspace_bytes) {
  THB_TIMED(stream, "thb200_gemm");
  cudaStream_t st = (cudaStream_t)stream;
  const bool ta = (transa == 't' || transa == 'T'), tb = (transb == 't' || transb == 'T');
  if (!ta && transa != 'n' && transa != 'N') return fail("gemm: transa must be 'n' or 't'");
  if (!tb && transb != 'n' && transb != 'N') return fail("gemm: transb must be 'n' or 't'");
  if (m < 0 || n < 0 || k < 0 || batch < 0) return fail("gemm: negative extent");
  if (m == 0 || n == 0 || batch == 0) return 0;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX || batch > 65535) return fail("gemm: extent too large");
  if (!a || !b || !c) return fail("gemm: null operand");
  if (lda < (ta ? k : m) || ldb < (tb ? n : k) || ldc < m)
    return fail("gemm: leading dimension too small (lda=%lld ldb=%lld ldc=%lld)", (long long)lda, (long long)ldb, (long long)ldc);
  Workspace w = carve(workspace, m, n, k > 0 ? k : 1, batch);
  if (!workspace || workspace_bytes < w.bytes)
    return fail("gemm: workspace too small (%zu bytes, need %zu)", workspace_bytes, w.bytes);

  const int64_t Kp = round_up(k > 0 ? k : 1, kKPad);
  // Three ways to get hi/lo operands to the tensor core:
  //  pre-pass  both operands are split in HBM first (12 bytes moved per operand element); the main
  //            loop then runs at ~0.9 of the tensor pipe. Any layout.
  //  fused     both operands are read in place and split in shared memory: nothing extra crosses HBM,
  //            but the conversion traffic costs the main loop about 40 % of its speed. For problems
  //            where the pre-pass would cost as much as the product (short K, few rows).
  //  pair      the same on clusters of two CTAs (tcgen05 cta_group::2, 256 x 256 tiles): each CTA holds
  //            half of the B' tile, a third less shared-memory traffic per CTA. Chosen instead of
  //            "fused" whenever the problem has at least two row tiles.
  //  ts        A' is read in place (either orientation) and split into TENSOR memory, only B' is
  //            pre-split: the main loop is faster than with pre-split operands and the big operand of
  //            "few rows x large weight matrix" is not pre-processed. Needs a long K (one accumulator).
  // THB200_GEMM_MODE=prepass|fused|pair|ts pins the choice where it is eligible (tests, experiments).
  enum { MODE_PREPASS = 0, MODE_FUSED = 1, MODE_TS = 2, MODE_PAIR = 3 };
  static const int forced_mode = [] {
    const char* e = getenv("THB200_GEMM_MODE");
    if (!e) return -1;
    return !strcmp(e, "fused") ? (int)MODE_FUSED : !strcmp(e, "ts") ? (int)MODE_TS : !strcmp(e, "prepass") ? (int)MODE_PREPASS
           : !strcmp(e, "pair") ? (int)MODE_PAIR : -1;
  }();
  const bool a_raw_ok = k > 0 && raw_operand_ok(a, lda, batch, stride_a);
  const bool fused_ok = a_raw_ok && raw_operand_ok(b, ldb, batch, stride_b);
  const bool ts_ok = a_raw_ok;
  int mode = MODE_PREPASS;
  if (forced_mode == MODE_FUSED) mode = fused_ok ? MODE_FUSED : MODE_PREPASS;
  else if (forced_mode == MODE_PAIR) mode = fused_ok ? MODE_PAIR : MODE_PREPASS;
  else if (forced_mode == MODE_TS) mode = ts_ok ? MODE_TS : MODE_PREPASS;
  else if (forced_mode < 0) {
    const double t_pre = 12.0 * (double)batch * ((double)m * k + (double)n * k) / 6.0e12;
    const double t_mma = 2.0 * (double)batch * (double)m * n * k / 250.0e12;
    if (ts_ok && k >= 1024) mode = MODE_TS;
    else if (fused_ok && t_pre > 0.3 * t_mma) mode = m > THB_GEMM_BM ? MODE_PAIR : MODE_FUSED;   // pairs need two row tiles
  }
  const bool pair = mode == MODE_PAIR;
  const bool fused = mode == MODE_FUSED || pair, ts = mode == MODE_TS;
  // op(A)(i, kk): column-major A, 'n': a[i + kk*lda] (unit stride along i), 't': a[kk + i*lda]
  if (mode == MODE_PREPASS) {
    dim3 grid((unsigned)(Kp / 32), (unsigned)((m + 31) / 32), (unsigned)batch);
    const bool rows_v4 = ta && ((uintptr_t)a & 15) == 0 && (lda & 3) == 0 && (batch == 1 || (stride_a & 3) == 0);
    if (rows_v4) {
      dim3 g4((unsigned)((Kp + 127) / 128), (unsigned)((m + 7) / 8), (unsigned)batch);
      thb_gemm_split_rows_v4<<<g4, 256, 0, st>>>(a, lda, stride_a, w.a, (int)m, (int)k, (int)Kp);
    } else if (!ta) thb_gemm_split<true><<<grid, 256, 0, st>>>(a, 1, lda, stride_a, w.a, (int)m, (int)k, (int)Kp);
    else thb_gemm_split<false><<<grid, 256, 0, st>>>(a, lda, 1, stride_a, w.a, (int)m, (int)k, (int)Kp);
    THB_CUDA(cudaGetLastError());
  }
  // B' row j, column kk = op(B)(kk, j): 'n': b[kk + j*ldb] (unit stride along kk), 't': b[j + kk*ldb]
  if (!fused) {
    dim3 grid((unsigned)(Kp / 32), (unsigned)((n + 31) / 32), (unsigned)batch);
    const bool rows_v4 = !tb && ((uintptr_t)b & 15) == 0 && (ldb & 3) == 0 && (batch == 1 || (stride_b & 3) == 0);
    if (rows_v4) {
      dim3 g4((unsigned)((Kp + 127) / 128), (unsigned)((n + 7) / 8), (unsigned)batch);
      thb_gemm_split_rows_v4<<<g4, 256, 0, st>>>(b, ldb, stride_b, w.b, (int)n, (int)k, (int)Kp);
    } else if (!tb) thb_gemm_split<false><<<grid, 256, 0, st>>>(b, ldb, 1, stride_b, w.b, (int)n, (int)k, (int)Kp);
    else thb_gemm_split<true><<<grid, 256, 0, st>>>(b, 1, ldb, stride_b, w.b, (int)n, (int)k, (int)Kp);
    THB_CUDA(cudaGetLastError());
  }
  THB_CUDA(cudaMemsetAsync(w.status, 0, sizeof(int), st));

  // k-block depth: 32 floats (128-byte swizzle, 2-stage ring) or 16 floats (64-byte swizzle,
  // 4-stage ring: more loads in flight). THB200_GEMM_BK overrides the default for experiments.
  static const int bk_default = [] {
    const char* e = getenv("THB200_GEMM_BK");
    return (e && atoi(e) == 32) ? 32 : 16;
  }();
  int bk = bk_default;
  // 128 x 128 tiles only when they finish sooner: a CTA works through ceil(tiles / SMs) tiles one
  // after the other, and a 128-wide tile takes about 0.8 of the time of a 256-wide one (half the
  // MMA columns, but the same A traffic and a lower tensor-pipe duty: measured 52% against 84%).
  const int sms = sm_count();
  const int64_t tm = (m + THB_GEMM_BM - 1) / THB_GEMM_BM;
  const int64_t tiles256 = tm * ((n + 255) / 256) * batch, tiles128 = tm * ((n + 127) / 128) * batch;
  static const int forced_bn = [] {  // THB200_GEMM_BN=128|256 pins the tile width (tests, experiments)
    const char* e = getenv("THB200_GEMM_BN");
    const int v = e ? atoi(e) : 0;
    return (v == 128 || v == 256) ? v : 0;
  }();
  const double cost256 = (double)((tiles256 + sms - 1) / sms), cost128 = 0.8 * (double)((tiles128 + sms - 1) / sms);
  // Split-K: when the 128 x 256 tiles fill at most half of the SMs and K is long, every tile is
  // cut along K into `splits` work items whose partial sums a small kernel adds up in a fixed order.
  static const int forced_splits = [] {  // THB200_GEMM_SPLITK=1..4 pins the split count (tests, experiments)
    const char* e = getenv("THB200_GEMM_SPLITK");
    const int v = e ? atoi(e) : 0;
    return (v >= 1 && v <= kMaxSplits) ? v : 0;
  }();
  int splits = 1;
  if (fused || ts) bk = 16;
  const int64_t kblocks_all = (fused || ts) ? (k + bk - 1) / bk : Kp / bk;
  if (tiles256 <= kSplitTileLimit && Kp >= 1024 && !forced_bn) {
    int64_t want = forced_splits ? forced_splits : sms / tiles256;
    if (want > kMaxSplits) want = kMaxSplits;
    if (want > kblocks_all / 32) want = kblocks_all / 32;   // at least 32 k blocks per split
    if (want >= 2 && (forced_splits || (double)((tiles256 * want + sms - 1) / sms) / (double)want + 0.1 < (cost128 < cost256 ? cost128 : cost256)))
      splits = (int)want;
  }
  int64_t kb_per_split = (kblocks_all + splits - 1) / splits;
  splits = (int)((kblocks_all + kb_per_split - 1) / kb_per_split);  // no empty split
  const int bn = pair ? 256 : (forced_bn ? forced_bn : (splits > 1 ? 256 : (cost128 < cost256 ? 128 : 256)));
  CUtensorMap map_a, map_b;
  // in memory, op(A) has unit stride along its rows for 'n' and along k for 't'; B' the other way round
  const bool a_mn = !ta, b_mn = tb;
  if (fused) {
    if (int rc = make_raw_operand_map(&map_a, a, a_mn, m, k, lda, batch, stride_a, THB_GEMM_BM, bk)) return rc;
    // a CTA of a pair loads only its half (128 rows) of a 256-row B' tile
    if (int rc = make_raw_operand_map(&map_b, b, b_mn, n, k, ldb, batch, stride_b, pair ? 128 : bn, bk)) return rc;
  } else if (ts) {
    if (a_mn) { if (int rc = make_raw_rows_map(&map_a, a, m, k, lda, batch, stride_a, bk)) return rc; }
    else if (int rc = make_raw_operand_map(&map_a, a, false, m, k, lda, batch, stride_a, THB_GEMM_BM, bk)) return rc;
    if (int rc = make_operand_map(&map_b, w.b, n, Kp, 2 * batch, bn, bk)) return rc;
  } else {
    if (int rc = make_operand_map(&map_a, w.a, m, Kp, 2 * batch, THB_GEMM_BM, bk)) return rc;
    if (int rc = make_operand_map(&map_b, w.b, n, Kp, 2 * batch, bn, bk)) return rc;
  }

  ThbGemmParams p;
  p.c = c;
  p.ldc = ldc;
  p.batch_stride_c = stride_c;
  p.m = (int)m;
  p.n = (int)n;
  p.kblocks = (int)kblocks_all;  // k == 0 (never fused): the split wrote zeros, so C = beta * C
  p.alpha = alpha;
  p.beta = beta;
  p.tiles_m = pair ? (int)((tm + 1) / 2) : (int)tm;   // pairs of CTAs take 256-row double tiles
  p.tiles_n = (int)((n + bn - 1) / bn);
  p.batch = (int)batch;
  p.status = w.status;
  p.splits = splits;
  p.kb_per_split = (int)kb_per_split;
  p.partial = w.partial;
  p.partial_split_stride = batch * m * n;
  const int64_t total_tiles = (int64_t)p.tiles_m * p.tiles_n * batch * splits;
  if (total_tiles > INT32_MAX) return fail("gemm: too many tiles");
  const unsigned ctas = pair ? 2u * (unsigned)(total_tiles < sms / 2 ? total_tiles : sms / 2)
                             : (unsigned)(total_tiles < sms ? total_tiles : sms);
  // 8 epilogue warps with the old C prefetched one block ahead: measured 0.181 ms against 0.230 ms
  // with 4 warps and no prefetch on the batched K = 128 shape, and no slower anywhere else
#define THB_LAUNCH_GEMM(BN_, BK_, ST_)                                                                                   \
  do {                                                                                                                   \
    THB_CUDA(cudaFuncSetAttribute(thb_gemm_3xtf32<BN_, BK_, ST_, 8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                  ThbGemmCfg<BN_, BK_, ST_>::kSmem));                                                    \
    thb_gemm_3xtf32<BN_, BK_, ST_, 8, true><<<ctas, THB_GEMM_THREADS(8), ThbGemmCfg<BN_, BK_, ST_>::kSmem, st>>>(        \
        map_a, map_b, p);                                                                                                \
  } while (0)
#define THB_LAUNCH_FUSED(BN_, ST_, AMN_, BMN_)                                                                             \
  do {                                                                                                                   \
    THB_CUDA(cudaFuncSetAttribute(thb_gemm_3xtf32_fused<BN_, 16, ST_, AMN_, BMN_>,                                        \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, ThbGemmFusedCfg<BN_, 16, ST_>::kSmem));   \
    thb_gemm_3xtf32_fused<BN_, 16, ST_, AMN_, BMN_>                                                                       \
        <<<ctas, THB_GEMM_FUSED_THREADS, ThbGemmFusedCfg<BN_, 16, ST_>::kSmem, st>>>(map_a, map_b, p);                    \
  } while (0)
#define THB_LAUNCH_FUSED_BN(AMN_, BMN_)                    \
  do {                                                     \
    if (bn == 256) THB_LAUNCH_FUSED(256, 4, AMN_, BMN_);   \
    else THB_LAUNCH_FUSED(128, 6, AMN_, BMN_);             \
  } while (0)
  if (ts) {
#define THB_LAUNCH_TS(BN_, ST_, AK_)                                                                                      \
  do {                                                                                                                   \
    THB_CUDA(cudaFuncSetAttribute(thb_gemm_3xtf32_ts<BN_, 16, ST_, AK_>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                  ThbGemmTsCfg<BN_, 16, ST_>::kSmem));                                                    \
    thb_gemm_3xtf32_ts<BN_, 16, ST_, AK_><<<ctas, THB_GEMM_TS_THREADS, ThbGemmTsCfg<BN_, 16, ST_>::kSmem, st>>>(map_a, map_b, p); \
  } while (0)
    if (bn == 256) { if (a_mn) THB_LAUNCH_TS(256, 5, false); else THB_LAUNCH_TS(256, 5, true); }
    else { if (a_mn) THB_LAUNCH_TS(128, 8, false); else THB_LAUNCH_TS(128, 8, true); }
#undef THB_LAUNCH_TS
  } else if (pair) {
#define THB_LAUNCH_PAIR(AMN_, BMN_)                                                                                       \
  do {                                                                                                                   \
    THB_CUDA(cudaFuncSetAttribute(thb_gemm_3xtf32_pair<16, 6, AMN_, BMN_>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                  ThbGemmPairCfg<16, 6>::kSmem));                                                          \
    thb_gemm_3xtf32_pair<16, 6, AMN_, BMN_><<<ctas, THB_GEMM_FUSED_THREADS, ThbGemmPairCfg<16, 6>::kSmem, st>>>(map_a, map_b, p); \
  } while (0)
    if (a_mn && b_mn) THB_LAUNCH_PAIR(true, true);
    else if (a_mn) THB_LAUNCH_PAIR(true, false);
    else if (b_mn) THB_LAUNCH_PAIR(false, true);
    else THB_LAUNCH_PAIR(false, false);
#undef THB_LAUNCH_PAIR
  } else if (fused) {
    if (a_mn && b_mn) THB_LAUNCH_FUSED_BN(true, true);
    else if (a_mn) THB_LAUNCH_FUSED_BN(true, false);
    else if (b_mn) THB_LAUNCH_FUSED_BN(false, true);
    else THB_LAUNCH_FUSED_BN(false, false);
  } else if (bn == 256 && bk == 32) THB_LAUNCH_GEMM(256, 32, 2);
  else if (bn == 256) THB_LAUNCH_GEMM(256, 16, 4);
  else if (bk == 32) THB_LAUNCH_GEMM(128, 32, 3);
  else THB_LAUNCH_GEMM(128, 16, 6);
#undef THB_LAUNCH_GEMM
#undef THB_LAUNCH_FUSED_BN
#undef THB_LAUNCH_FUSED
  THB_CUDA(cudaGetLastError());
  if (splits > 1) {
    const bool vec = (m & 3) == 0 && (ldc & 3) == 0 && (stride_c & 3) == 0 && ((uintptr_t)c & 15) == 0;
    dim3 grid((unsigned)((m / (vec ? 4 : 1) + 255) / 256), (unsigned)((n + 3) / 4), (unsigned)batch);
    if (vec) thb_gemm_splitk_fixup<true><<<grid, 256, 0, st>>>(c, ldc, stride_c, w.partial, p.partial_split_stride, splits, (int)m, (int)n, alpha, beta);
    else thb_gemm_splitk_fixup<false><<<grid, 256, 0, st>>>(c, ldc, stride_c, w.partial, p.partial_split_stride, splits, (int)m, (int)n, alpha, beta);
    THB_CUDA(cudaGetLastError());
  }
  return 0;
}

/* Status word of the last thb200_gemm on this workspace: 0 = completed,
 * 1/2/3 = a bounded wait of the producer / MMA issuer / epilogue gave up.
 * Synchronises the stream. */
int thb200_gemm_status(void* stream, int64_t m, int64_t n, int64_t k, int64_t batch, void* workspace) {
  Workspace w = carve(workspace, m, n, k > 0 ? k : 1, batch);
  int h = -1;
  if (cudaMemcpyAsync(&h, w.status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess ||
      cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) {
    fail("gemm: could not read the status word");
    return -1;
  }
  return h;
}

}  // extern "C"
