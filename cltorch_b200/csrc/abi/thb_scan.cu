// Host side of the scans, renorm and dist entries of include/thb200.h.
#include "thb_internal.h"
#include "../kernels/math_policy.cuh"
#include "../kernels/scan_strip_kernels.cuh"
#include "../kernels/scan_chain_kernels.cuh"
#include "../kernels/renorm_kernels.cuh"

#define THB_SCH_TILE 8192  // elements per tile of the chained scan
// 3 stages of first visits, 4 of second visits, at most 6 tiles between the two, first visits loaded with the
// L2 evict-last priority, second visits and results with evict-first: 342-344 us on 2^28 elements. Without the
// priorities: 349-352 us with at most 4 tiles between the visits (3/3/4 stages 363 us, 2/4/4 385 us, 3/3/3
// 414 us) and 423-480 us with 5 or more (a longer lead of the first visits then pushes tiles out of L2 before
// their second visit); with them 346 us at 5, 366 us at 8.
#define THB_SCH_SA 3
#define THB_SCH_SB 4
#define THB_SCH_NSLOT 6
#include "thb_strips.h"

namespace thb {

struct ScanPlan {
  bool rows;        // inner == 1
  int vec;          // 4 or 1
  uint32_t nchunks, chunk_len;
  bool strips;      // single pass over 128-column strips through a TMA pipeline
  int strips_per_outer, total_strips;
  bool chain;       // inner == 1, few long rows: single pass over tiles that wait for their carries
  uint32_t tail;    // chain, one vector: elements after the last multiple of 32, scanned by a follow-up kernel
};

static size_t scan_scratch_need(const ScanPlan& p, int64_t outer, int64_t inner) {
  if (p.nchunks <= 1) return 0;
  return ((size_t)outer * p.nchunks * inner + (p.chain ? (size_t)outer : 0)) * sizeof(double);
}

// Whether the chained scan can run here: kernels can be launched with all their CTAs guaranteed resident
// (its CTAs wait for one another's totals) and one CTA of it fits on an SM.
static bool cooperative_launch_ok() {
  static int cached[64];  // 0 unknown, 1 yes, 2 no
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  if (!cached[dev]) {
    int v = 0, per_sm = 0;
    auto kern = thb_scan_chain<ScanAdd, THB_SCH_TILE, THB_SCH_SA, THB_SCH_SB, THB_SCH_NSLOT, 3>;
    const int smem = THB_SCH_SMEM_BYTES(THB_SCH_TILE, THB_SCH_SA, THB_SCH_SB, THB_SCH_NSLOT);
    const bool ok = cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && v &&
                    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THB_SCH_THREADS, smem) == cudaSuccess &&
                    per_sm >= 1;
    if (!ok) cudaGetLastError();
    cached[dev] = ok ? 1 : 2;
  }
  return cached[dev] == 1;
}

static ScanPlan plan_scan(const float* dst, const float* src, int64_t outer, int64_t n, int64_t inner) {
  ScanPlan p;
  p.strips = false;
  p.strips_per_outer = p.total_strips = 0;
  p.chain = false;
  p.tail = 0;
  p.rows = inner == 1;
  const bool aligned = (((uintptr_t)dst | (uintptr_t)src) & 15) == 0;
  if (p.rows) {
    p.vec = (aligned && (n & 3) == 0) ? 4 : 1;
    const int64_t piece = 32 * p.vec * THB_SC_ROW_UNROLL;  // elements one warp step covers
    // one warp per (row, chunk): aim at 8 blocks of 8 warps per SM, chunks of at least 4 pieces
    const int64_t target_warps = (int64_t)sm_count() * 64;
    int64_t chunks = outer * 2 > target_warps ? 1 : target_warps / outer;
    const int64_t max_chunks = n / (4 * piece);
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    int64_t len = (n + chunks - 1) / chunks;
    len = (len + piece - 1) / piece * piece;
    p.chunk_len = (uint32_t)len;
    p.nchunks = (uint32_t)((n + len - 1) / len);
    // Rows that have to be cut (three phases, 12 bytes per element) go through the chained single-pass
    // kernel instead when the layout suits TMA: 349 against 621 us on one vector of 2^28 elements. With enough
    // rows for a warp per row the two are level (16384 rows of 16384: 352 against 362 us over ten calls, but
    // 389 against 372 us in a 0.25 s loop under the power cap), so those keep the warp per row.
    if (p.nchunks > 1 && aligned && ((n & 31) == 0 || outer == 1) && n >= 2 * THB_SCH_TILE &&
        outer < (int64_t(1) << 31) && cooperative_launch_ok() && tensor_map_encoder_ptr() != nullptr) {
      p.chain = true;
      p.tail = (uint32_t)(n & 31);
      p.chunk_len = THB_SCH_TILE;
      p.nchunks = (uint32_t)((n - p.tail + THB_SCH_TILE - 1) / THB_SCH_TILE);
    }
  } else {
    p.vec = (aligned && (inner & 3) == 0) ? 4 : 1;
    p.nchunks = pick_chunks(outer * inner / p.vec, n, THB_SC_COLS_BLOCKS);
    p.chunk_len = (uint32_t)((n + p.nchunks - 1) / p.nchunks);
    // Where the one-thread-per-column kernel would have to cut the rows into chunks (three
    // phases, 12 bytes per element), a strip per CTA does it in one pass, provided there are
    // enough strips to keep HBM busy and the layout suits TMA (16-byte aligned rows).
    const int64_t spo = (inner + THB_SS_COLS - 1) / THB_SS_COLS;
    const int64_t total = spo * outer;
    // One strip per CTA sustains about 50 GB/s (a column is one thread's chain of fp64 additions
    // and conversions), so it takes strips on two thirds of the SMs to beat the chunked kernels:
    // measured at 8192 columns (64 strips) 159 us against 143 us, at 16384 (128 strips) 0.35 ms
    // against 0.55 ms.
    if (p.nchunks > 1 && aligned && (inner & 3) == 0 && total * 3 >= (int64_t)sm_count() * 2 &&
        total < (int64_t(1) << 31) &&
        n >= 2 * THB_SS_ROWS && inner < (int64_t(1) << 31) && outer < (int64_t(1) << 31) &&
        n * inner * 4 < (int64_t(1) << 40) && tensor_map_encoder_ptr() != nullptr) {
      p.strips = true;
      p.strips_per_outer = (int)spo;
      p.total_strips = (int)total;
      p.nchunks = 1;  // no carries, no scratch
    }
  }
  return p;
}

template <class Op>
static int run_scan_strips(cudaStream_t st, float* dst, const float* src, int64_t outer, int64_t n, int64_t inner,
                           const ScanPlan& p, int* d_status) {
  CUtensorMap map_src, map_dst;
  if (int rc = make_strip_map(&map_src, src, outer, n, inner, inner)) return rc;
  if (int rc = make_strip_map(&map_dst, dst, outer, n, inner, inner)) return rc;
  THB_CUDA(cudaFuncSetAttribute(thb_scan_strips<Op>, cudaFuncAttributeMaxDynamicSharedMemorySize, THB_SS_SMEM));
  const int sms = sm_count();
  const int ctas = p.total_strips < sms ? p.total_strips : sms;
  thb_scan_strips<Op><<<ctas, THB_SCAN_STRIP_THREADS, THB_SS_SMEM, st>>>(map_src, map_dst, (thb_u32)n, inner, p.strips_per_outer,
                                                                          p.total_strips, d_status ? d_status : device_status_word(STATUS_STRIP_SCAN));
  THB_CUDA(cudaGetLastError());
  return 0;
}

// Tensor map over [outer][n / 32][32] floats with the 128-byte swizzle: a box is one tile of the chained scan.
static int make_chain_map(CUtensorMap* map, const float* p, int64_t outer, int64_t n) {
  auto enc = (PFN_cuTensorMapEncodeTiled_v12000)tensor_map_encoder_ptr();
  cuuint64_t dims[3] = {32, (cuuint64_t)(n / 32), (cuuint64_t)outer};
  cuuint64_t strides[2] = {128, (cuuint64_t)n * 4};
  cuuint32_t box[3] = {32, THB_SCH_TILE / 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)p, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("scan: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

template <class Op>
static int run_scan_chain(cudaStream_t st, float* dst, const float* src, int64_t outer, int64_t n, double* scratch,
                          const ScanPlan& p, int* d_status) {
  thb_i64 nwork = outer * (int64_t)p.nchunks;
  unsigned long long* totals = (unsigned long long*)scratch;
  double* row_carry = scratch + nwork;  // [outer]
  const int64_t n_all = n;
  n -= p.tail;  // the part the tiles cover
  THB_CUDA(cudaMemsetAsync(totals, 0xFF, (size_t)nwork * sizeof(unsigned long long), st));  // "not written yet"
  int ctas = sm_count() < THB_SCH_MAX_CTAS ? sm_count() : THB_SCH_MAX_CTAS;
  if (nwork < ctas) ctas = (int)nwork;
  thb_u32 n32 = (thb_u32)n, nchunks = p.nchunks;
  int* status = d_status ? d_status : device_status_word(STATUS_STRIP_SCAN);
  CUtensorMap map_src, map_dst;
  if (int rc = make_chain_map(&map_src, src, outer, n)) return rc;
  if (int rc = make_chain_map(&map_dst, dst, outer, n)) return rc;
  void* args[] = {&map_src, &map_dst, &n32, &nchunks, &nwork, &totals, &row_carry, &status};
  auto kern = thb_scan_chain<Op, THB_SCH_TILE, THB_SCH_SA, THB_SCH_SB, THB_SCH_NSLOT, 3>;
  const int smem = THB_SCH_SMEM_BYTES(THB_SCH_TILE, THB_SCH_SA, THB_SCH_SB, THB_SCH_NSLOT);
  THB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  THB_CUDA(cudaLaunchCooperativeKernel((const void*)kern, dim3(ctas), dim3(THB_SCH_THREADS), args, smem, st));
  if (p.tail) {
    thb_scan_chain_tail<Op><<<1, 32, 0, st>>>(dst, src, n32, (thb_u32)n_all, nchunks, totals, row_carry);
    THB_CUDA(cudaGetLastError());
  }
  return 0;
}

template <class Op>
static int run_scan(cudaStream_t st, float* dst, const float* src, int64_t outer, int64_t n, int64_t inner, double* carry,
                    const ScanPlan& p, int* d_status) {
  if (p.strips) return run_scan_strips<Op>(st, dst, src, outer, n, inner, p, d_status);
  if (p.chain) return run_scan_chain<Op>(st, dst, src, outer, n, carry, p, d_status);
  const int sms = sm_count();
  if (p.rows) {
    const int64_t work = outer * p.nchunks;  // warps
    int64_t blocks = (work + THB_SC_THREADS / 32 - 1) / (THB_SC_THREADS / 32);
    if (blocks > kMaxGridBlocks) blocks = kMaxGridBlocks;
    if (p.nchunks > 1) {
      if (p.vec == 4) thb_scan_rows<Op, 4, true><<<(unsigned)blocks, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, p.chunk_len, p.nchunks, carry);
      else thb_scan_rows<Op, 1, true><<<(unsigned)blocks, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, p.chunk_len, p.nchunks, carry);
      THB_CUDA(cudaGetLastError());
      if (p.nchunks >= 64) {  // few long rows: a block per row
        int64_t cb = outer < (int64_t)sms * 8 ? outer : (int64_t)sms * 8;
        thb_scan_carries_rows<Op><<<(unsigned)cb, THB_SC_THREADS, 0, st>>>(carry, outer, p.nchunks);
      } else {
        int64_t cb = (outer + 31) / 32;
        if (cb > kMaxGridBlocks) cb = kMaxGridBlocks;
        thb_scan_carries<Op><<<(unsigned)cb, THB_SC_THREADS, 0, st>>>(carry, outer, p.nchunks, 1);
      }
      THB_CUDA(cudaGetLastError());
    }
    if (p.vec == 4) thb_scan_rows<Op, 4, false><<<(unsigned)blocks, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, p.chunk_len, p.nchunks, carry);
    else thb_scan_rows<Op, 1, false><<<(unsigned)blocks, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, p.chunk_len, p.nchunks, carry);
    THB_CUDA(cudaGetLastError());
    return 0;
  }
  const int64_t threads = outer * inner / p.vec;
  int64_t bx = (threads + THB_SC_THREADS - 1) / THB_SC_THREADS;
  if (bx > kMaxGridBlocks) bx = kMaxGridBlocks;
  const dim3 grid((unsigned)bx, p.nchunks);
  if (p.nchunks > 1) {
    if (p.vec == 4) thb_scan_cols<Op, 4, true><<<grid, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, inner, p.chunk_len, p.nchunks, carry);
    else thb_scan_cols<Op, 1, true><<<grid, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, inner, p.chunk_len, p.nchunks, carry);
    THB_CUDA(cudaGetLastError());
    int64_t cb = (outer * inner + 31) / 32;  // 32 positions x 8 lanes per block
    if (cb > kMaxGridBlocks) cb = kMaxGridBlocks;
    thb_scan_carries<Op><<<(unsigned)cb, THB_SC_THREADS, 0, st>>>(carry, outer, p.nchunks, inner);
    THB_CUDA(cudaGetLastError());
  }
  if (p.vec == 4) thb_scan_cols<Op, 4, false><<<grid, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, inner, p.chunk_len, p.nchunks, carry);
  else thb_scan_cols<Op, 1, false><<<grid, THB_SC_THREADS, 0, st>>>(dst, src, outer, (thb_u32)n, inner, p.chunk_len, p.nchunks, carry);
  THB_CUDA(cudaGetLastError());
  return 0;
}

// Rows that fit in the registers of a warp or of a CTA are renormed in one pass.
template <int PMODE>
static bool launch_renorm_fused(cudaStream_t st, float* data, int64_t rows, int64_t size, float p, float maxnorm) {
  const int64_t nvec = size / 4;
  const int sms = sm_count();
  const thb_u32 size32 = (thb_u32)size;
#define THB_RNF_WARP(L, U, R)                                                                                        \
  do {                                                                                                               \
    const int64_t per_block = (int64_t)(THB_RNF_THREADS / 32) * (R) * (32 / (L));                                    \
    int64_t blocks = (rows + per_block - 1) / per_block;                                                             \
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;                                                        \
    thb_renorm_rows_warp<L, U, R, PMODE><<<(unsigned)blocks, THB_RNF_THREADS, 0, st>>>(data, rows, size32, p, maxnorm); \
  } while (0)
#define THB_RNF_BLOCK(THREADS)                                                                                       \
  do {                                                                                                               \
    const int64_t resident = (int64_t)sms * (512 / (THREADS));                                                       \
    const int64_t blocks = rows < resident * 4 ? rows : resident * 4;                                                \
    thb_renorm_rows_block<THREADS, PMODE><<<(unsigned)blocks, THREADS, 0, st>>>(data, rows, size32, p, maxnorm);      \
  } while (0)
  if (nvec <= 8) THB_RNF_WARP(8, 1, 8);
  else if (nvec <= 16) THB_RNF_WARP(16, 1, 8);
  else if (nvec <= 32) THB_RNF_WARP(32, 1, 8);
  else if (nvec <= 64) THB_RNF_WARP(32, 2, 4);
  else if (nvec <= 128) THB_RNF_WARP(32, 4, 2);
  else if (nvec <= 256) THB_RNF_WARP(32, 8, 1);
  else if (nvec <= 512) THB_RNF_WARP(32, 16, 1);
  else if (nvec <= 64 * THB_RNF_BLOCK_U) THB_RNF_BLOCK(64);
  else if (nvec <= 128 * THB_RNF_BLOCK_U) THB_RNF_BLOCK(128);
  else if (nvec <= 256 * THB_RNF_BLOCK_U) THB_RNF_BLOCK(256);
  else return false;
#undef THB_RNF_WARP
#undef THB_RNF_BLOCK
  return true;
}

static int64_t dist_blocks(int64_t n) {
  const int64_t per_block = (int64_t)THB_RA_THREADS * 16;
  int64_t blocks = (n + per_block - 1) / per_block;
  if (blocks > THB_RA_MAX_BLOCKS) blocks = THB_RA_MAX_BLOCKS;
  return blocks < 1 ? 1 : blocks;
}

}  // namespace thb

using namespace thb;

extern "C" {

size_t thb200_scan_scratch_bytes(const float* dst, const float* src, int64_t outer, int64_t n, int64_t inner) {
  if (outer <= 0 || n <= 0 || inner <= 0) return 0;
  const ScanPlan p = plan_scan(dst, src, outer, n, inner);
  return scan_scratch_need(p, outer, inner);
}

int thb200_scan(void* stream, int op, float* dst, const float* src, int64_t outer, int64_t n, int64_t inner,
                void* scratch, size_t scratch_bytes, int* d_status) {
  THB_TIMED(stream, "thb200_scan");
  if (outer < 0 || n < 0 || inner < 0) return fail("scan: negative extent");
  if (outer == 0 || n == 0 || inner == 0) return 0;
  if (!dst || !src) return fail("scan: null pointer");
  if (n >= (int64_t(1) << 31)) return fail("scan: dimension of %lld elements is too long", (long long)n);
  if (op != THB200_RED_ADD && op != THB200_RED_MUL) return fail("scan: operator %d is neither add nor mul", op);
  const ScanPlan p = plan_scan(dst, src, outer, n, inner);
  const size_t need = scan_scratch_need(p, outer, inner);
  if (need && (!scratch || scratch_bytes < need || ((uintptr_t)scratch & 7)))
    return fail("scan: scratch too small or misaligned (%zu bytes, need %zu)", scratch_bytes, need);
  return op == THB200_RED_ADD
             ? run_scan<ScanAdd>((cudaStream_t)stream, dst, src, outer, n, inner, (double*)scratch, p, d_status)
             : run_scan<ScanMul>((cudaStream_t)stream, dst, src, outer, n, inner, (double*)scratch, p, d_status);
}

size_t thb200_renorm_rows_scratch_bytes(int64_t rows, int64_t size) {
  if (rows <= 0 || size <= 0) return 0;
  return (size_t)rows * sizeof(float);
}

int thb200_renorm_rows(void* stream, float* data, int64_t rows, int64_t size, float p, float maxnorm, void* scratch,
                       size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_renorm_rows");
  if (rows < 0 || size < 0) return fail("renorm: negative extent");
  if (rows == 0 || size == 0) return 0;
  if (!data) return fail("renorm: null pointer");
  if (!(p > 0.f)) return fail("renorm: non-positive-norm not supported");
  if (rows >= (int64_t(1) << 31) || size >= (int64_t(1) << 31)) return fail("renorm: extent too large");
  if (!scratch || scratch_bytes < (size_t)rows * sizeof(float)) return fail("renorm: scratch too small");
  if ((((uintptr_t)data) & 15) == 0 && (size & 3) == 0 && size <= 4 * 256 * THB_RNF_BLOCK_U) {
    cudaStream_t st = (cudaStream_t)stream;
    const bool done = p == 1.0f   ? launch_renorm_fused<1>(st, data, rows, size, p, maxnorm)
                      : p == 2.0f ? launch_renorm_fused<2>(st, data, rows, size, p, maxnorm)
                      : p == 3.0f ? launch_renorm_fused<3>(st, data, rows, size, p, maxnorm)
                                  : launch_renorm_fused<0>(st, data, rows, size, p, maxnorm);
    if (done) {
      THB_CUDA(cudaGetLastError());
      return 0;
    }
  }
  // sum |x|^p of every row: the contiguous-dimension reduction, [rows][size] -> [rows][1]
  const int64_t in_size[2] = {rows, size}, in_stride[2] = {size, 1};
  const int64_t out_size[2] = {rows, 1}, out_stride[2] = {1, 1};
  thb200_tensor tin = {data, 2, in_size, in_stride}, tout = {(float*)scratch, 2, out_size, out_stride};
  if (int rc = thb200_reduce_dim(stream, THB200_MOD_ABSPOW, THB200_RED_ADD, &tout, &tin, 1, 0.f, p, nullptr, 0)) return rc;
  const int64_t pieces = (size + THB_RN_PIECE - 1) / THB_RN_PIECE;
  int64_t blocks = rows * pieces;
  const int64_t cap = kMaxGridBlocks;
  if (blocks > cap) blocks = cap;
  thb_renorm_scale<<<(unsigned)blocks, THB_SC_THREADS, 0, (cudaStream_t)stream>>>(data, (const float*)scratch, rows, size, p,
                                                                                   maxnorm, pieces);
  THB_CUDA(cudaGetLastError());
  return 0;
}

size_t thb200_dist_scratch_bytes(int64_t n) { return (size_t)dist_blocks(n) * sizeof(double); }

int thb200_dist(void* stream, const float* a, const float* b, int64_t n, float p, float* d_out, void* scratch,
                size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_dist");
  if (n < 0) return fail("dist: negative length");
  if (!d_out) return fail("dist: null output");
  if (n > 0 && (!a || !b)) return fail("dist: null pointer");
  const int blocks = (int)dist_blocks(n);
  if (!scratch || scratch_bytes < (size_t)blocks * sizeof(double) || ((uintptr_t)scratch & 7))
    return fail("dist: scratch too small or misaligned");
  const int vec_ok = (((uintptr_t)a | (uintptr_t)b) & 15) == 0;
  thb_dist_pass1<<<blocks, THB_RA_THREADS, 0, (cudaStream_t)stream>>>(a, b, n, p, vec_ok, (double*)scratch);
  THB_CUDA(cudaGetLastError());
  thb_dist_pass2<<<1, 1024, 0, (cudaStream_t)stream>>>((const double*)scratch, blocks, p, d_out);
  THB_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
