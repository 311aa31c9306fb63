// Host side of thb200_dot and thb200_gemv.
#include "thb_internal.h"
#include "../kernels/math_policy.cuh"
#include "../kernels/blas_kernels.cuh"
#include "thb_strips.h"

using namespace thb;

extern "C" {

size_t thb200_dot_scratch_bytes(int64_t n) {
  (void)n;
  return (size_t)THB_RA_MAX_BLOCKS * sizeof(double);
}

int thb200_dot(void* stream, const float* a, const float* b, int64_t n, float* d_out, void* scratch,
               size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_dot");
  if (n < 0) return fail("dot: negative length");
  if (!d_out) return fail("dot: null output");
  if (n > 0 && (!a || !b)) return fail("dot: null operand");
  if (!scratch || scratch_bytes < thb200_dot_scratch_bytes(n)) return fail("dot: scratch too small");
  cudaStream_t st = (cudaStream_t)stream;
  int64_t per_block = (int64_t)THB_RA_THREADS * 16;
  int64_t blocks = (n + per_block - 1) / per_block;
  if (blocks > THB_RA_MAX_BLOCKS) blocks = THB_RA_MAX_BLOCKS;
  if (blocks < 1) blocks = 1;
  const int vec_ok = ((((uintptr_t)a) | ((uintptr_t)b)) & 15) == 0;
  ThbFinish F;
  F.ticket = reduce_ticket();
  F.fin = THB_FIN_NONE; F.fparam = 1.f; F.out = d_out;
  thb_dot_pass1<<<(unsigned)blocks, THB_RA_THREADS, 0, st>>>(a, b, n, vec_ok, (double*)scratch, F);
  THB_CUDA(cudaGetLastError());
  if (!F.ticket) {
    thb_reduce_all_pass2<RedAdd><<<1, 1024, 0, st>>>((const double*)scratch, (int)blocks, 0.f, THB_FIN_NONE, 1.f, d_out);
    THB_CUDA(cudaGetLastError());
  }
  return 0;
}

static uint32_t gemv_chunks(int64_t m, int64_t n) {
  const int64_t want = (int64_t)sm_count() * 2048;
  if (m >= want || n < 256) return 1;
  int64_t chunks = (want + m - 1) / m;
  if (chunks > n / 64) chunks = n / 64;
  if (chunks > 1024) chunks = 1024;
  return (uint32_t)(chunks < 1 ? 1 : chunks);
}

// Two threads per output in the strip path: two partials per output and chunk.
static const int kGemvHalves = 2;

size_t thb200_gemv_scratch_bytes(char trans, int64_t m, int64_t n) {
  if (trans == 't' || trans == 'T' || m <= 0 || n <= 0) return 0;
  uint32_t c = gemv_chunks(m, n);
  size_t plain = c > 1 ? (size_t)c * m * sizeof(double) : 0;
  // the strip path is taken when A is 16-byte aligned with lda a multiple of 4: size for whichever needs more
  const StripPlan sp = plan_strips(nullptr, 1, n, m);
  size_t strips = sp.ok ? (size_t)kGemvHalves * sp.nchunks * m * sizeof(double) : 0;
  return strips > plain ? strips : plain;
}

int thb200_gemv(void* stream, char trans, int64_t m, int64_t n, float alpha, const float* a, int64_t lda, const float* x,
                int64_t incx, float beta, float* y, int64_t incy, void* scratch, size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_gemv");
  const bool t = (trans == 't' || trans == 'T');
  if (!t && trans != 'n' && trans != 'N') return fail("gemv: trans must be 'n' or 't'");
  if (m < 0 || n < 0) return fail("gemv: negative extent");
  if (m > UINT32_MAX || n > UINT32_MAX) return fail("gemv: extent too large");
  if (lda < (m > 1 ? m : 1)) return fail("gemv: lda %lld < m %lld", (long long)lda, (long long)m);
  const int64_t ylen = t ? n : m;
  if (ylen == 0) return 0;
  if (!a || !x || !y) return fail("gemv: null operand");
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = sm_count();
  if (t) {
    // y (n) = alpha * A^T x + beta * y: one contiguous column of A (length m) per output
    if (m < 8192) {
      int64_t blocks = (n + 7) / 8;
      if (blocks > kMaxGridBlocks) blocks = kMaxGridBlocks;
      thb_gemv_t<true><<<(unsigned)blocks, THB_RD_THREADS, 0, st>>>(a, lda, x, incx, y, incy, (thb_u32)m, (thb_u32)n, alpha, beta);
    } else {
      int64_t blocks = n < kMaxGridBlocks ? n : kMaxGridBlocks;
      thb_gemv_t<false><<<(unsigned)blocks, THB_RD_THREADS, 0, st>>>(a, lda, x, incx, y, incy, (thb_u32)m, (thb_u32)n, alpha, beta);
    }
    THB_CUDA(cudaGetLastError());
    return 0;
  }
  int64_t bxf = (m + THB_RD_THREADS - 1) / THB_RD_THREADS;
  if (bxf > 65535 * 16) bxf = 65535 * 16;
  const StripPlan sp = (lda & 3) == 0 ? plan_strips(a, 1, n, m) : StripPlan();
  if (sp.ok && lda * n * 4 < (int64_t(1) << 40)) {
    // y(m) = alpha * A x + beta * y: strips of 128 outputs, the columns of A stream by as rows
    const uint32_t nparts = kGemvHalves * sp.nchunks;
    if (!scratch || scratch_bytes < (size_t)nparts * m * sizeof(double) || ((uintptr_t)scratch & 7))
      return fail("gemv: scratch too small (%zu bytes, need %zu)", scratch_bytes, (size_t)nparts * m * sizeof(double));
    CUtensorMap map;
    if (int rc = make_strip_map(&map, a, 1, n, m, lda)) return rc;
    ThbStripGeom g;
    g.n = (thb_u32)n; g.inner = m; g.strips_per_outer = sp.strips_per_outer; g.total_strips = sp.total_strips;
    g.nchunks = sp.nchunks; g.chunk_rows = sp.chunk_rows; g.npartials = nparts; g.nslices = (thb_u32)m;
    ThbGemvConsumer::Params cp;
    cp.x = x; cp.incx = incx; cp.partial = (double*)scratch;
    THB_CUDA(cudaFuncSetAttribute(thb_strip_reduce<ThbGemvConsumer, kGemvHalves>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  THB_SS_SMEM));
    const int64_t items = (int64_t)sp.total_strips * sp.nchunks;
    const unsigned ctas = (unsigned)(items < sms ? items : sms);
    thb_strip_reduce<ThbGemvConsumer, kGemvHalves><<<ctas, 32 + 128 * kGemvHalves, THB_SS_SMEM, st>>>(map, g, cp,
                                                                                                      device_status_word(STATUS_STRIP_GEMV));
    THB_CUDA(cudaGetLastError());
    thb_gemv_n_fold<<<(unsigned)bxf, THB_RD_THREADS, 0, st>>>((const double*)scratch, y, incy, (thb_u32)m, nparts, alpha, beta);
    THB_CUDA(cudaGetLastError());
    return 0;
  }
  const uint32_t nchunks = gemv_chunks(m, n);
  const uint32_t chunk_len = (uint32_t)((n + nchunks - 1) / nchunks);
  if (nchunks > 1 && (!scratch || scratch_bytes < (size_t)nchunks * m * sizeof(double)))
    return fail("gemv: scratch too small (%zu bytes, need %zu)", scratch_bytes, (size_t)nchunks * m * sizeof(double));
  int64_t bx = (m + THB_RD_THREADS - 1) / THB_RD_THREADS;
  if (bx > 65535 * 16) bx = 65535 * 16;
  dim3 grid((unsigned)bx, nchunks ? nchunks : 1);
  thb_gemv_n<<<grid, THB_RD_THREADS, 0, st>>>(a, lda, x, incx, y, incy, (thb_u32)m, (thb_u32)n, alpha, beta, chunk_len,
                                             nchunks, (double*)scratch);
  THB_CUDA(cudaGetLastError());
  if (nchunks > 1) {
    thb_gemv_n_fold<<<(unsigned)bx, THB_RD_THREADS, 0, st>>>((const double*)scratch, y, incy, (thb_u32)m, nchunks, alpha, beta);
    THB_CUDA(cudaGetLastError());
  }
  return 0;
}

/* clblasSger as called from THClBlas_ger: column-major A (m x n, unit stride along m):
 * A[i + j*lda] += (alpha * y[j*incy]) * x[i], or (alpha * x[i]) * y[j*incy] with alpha_on_x.
 * Needs the 128-bit path: A and x 16-byte aligned,
 * x contiguous, m and lda multiples of 4; returns 1 (and does nothing) when the operands do not
 * qualify, so that the caller can fall back to the pointwise operator. */
int thb200_ger(void* stream, int64_t m, int64_t n, float alpha, const float* x, int64_t incx, const float* y, int64_t incy,
               float* a, int64_t lda, int alpha_on_x) {
  THB_TIMED(stream, "thb200_ger");
  if (m < 0 || n < 0) return fail("ger: negative extent");
  if (m == 0 || n == 0) return 0;
  if (!x || !y || !a) return fail("ger: null operand");
  if (incx != 1 || (m & 3) != 0 || (lda & 3) != 0 || lda < m || ((((uintptr_t)a) | ((uintptr_t)x)) & 15) != 0 ||
      m > UINT32_MAX || n > UINT32_MAX)
    return 1;
  const uint64_t nvec = (uint64_t)n * (uint64_t)(m >> 2);
  uint64_t blocks = (nvec + 1023) / 1024;
  const uint64_t cap = (uint64_t)kMaxGridBlocks;
  if (blocks > cap) blocks = cap;
  if (alpha_on_x)
    thb_ger_rows<false><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a, lda, (thb_u32)n, (thb_u32)(m >> 2), y, incy, x, alpha);
  else
    thb_ger_rows<true><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a, lda, (thb_u32)n, (thb_u32)(m >> 2), y, incy, x, alpha);
  THB_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
