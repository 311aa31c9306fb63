// Host side of the reductions in include/thb200.h: kernel selection, grid
// sizing and scratch layout.
#include "thb_internal.h"
#include "../kernels/math_policy.cuh"
#include "../kernels/reduce_kernels.cuh"
#include "../kernels/reduce_strip_kernels.cuh"
#include "thb_strips.h"

#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

namespace thb {

void fastdiv_constants_pub(uint32_t d, uint32_t* magic, uint32_t* shift) {
  uint32_t l = 0;
  while (l < 32 && (uint64_t(1) << l) < d) ++l;
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
    fastdiv_constants_pub((uint32_t)c.size[d], &L->magic[d], &L->shift[d]);
  }
}

static int64_t reduce_all_blocks(int64_t n) {
  int64_t per_block = (int64_t)THB_RA_THREADS * THB_RA_UNROLL * 4;
  int64_t pieces = (n + per_block - 1) / per_block;
  if (pieces < 1) pieces = 1;
  // every block takes the same number of pieces (a function of n alone, so the summation order
  // stays independent of the device): 2048 pieces run as 512 blocks x 4 rather than 592 blocks of
  // which three quarters take 3 and the rest 4
  const int64_t sweeps = (pieces + THB_RA_MAX_BLOCKS - 1) / THB_RA_MAX_BLOCKS;
  return (pieces + sweeps - 1) / sweeps;
}

// Calls f.template operator()<Mod, Red>() for the pair the reference's
// front-ends use; false for a pair nobody asks for.
template <class F>
static bool dispatch_pair(int modify, int reduce, float mod_param, F&& f) {
  switch (modify) {
    case THB200_MOD_COPY:
      switch (reduce) {
        case THB200_RED_ADD: f.template operator()<ModCopy, RedAdd>(); return true;
        case THB200_RED_MUL: f.template operator()<ModCopy, RedMul>(); return true;
        case THB200_RED_MIN: f.template operator()<ModCopy, RedMin>(); return true;
        case THB200_RED_MAX: f.template operator()<ModCopy, RedMax>(); return true;
        case THB200_RED_AND: f.template operator()<ModCopy, RedAnd>(); return true;
        case THB200_RED_OR: f.template operator()<ModCopy, RedOr>(); return true;
      }
      return false;
    case THB200_MOD_ABSPOW:
      if (reduce != THB200_RED_ADD) return false;
      if (mod_param == 2.0f) f.template operator()<ModSquare, RedAdd>();
      else if (mod_param == 1.0f) f.template operator()<ModAbs, RedAdd>();
      else if (mod_param == 3.0f) f.template operator()<ModAbsCube, RedAdd>();
      else f.template operator()<ModAbsPow, RedAdd>();
      return true;
    case THB200_MOD_NEZERO:
      if (reduce == THB200_RED_ADD) { f.template operator()<ModNeZero, RedAdd>(); return true; }
      return false;
    case THB200_MOD_SQDEV:
      if (reduce == THB200_RED_ADD) { f.template operator()<ModSqDev, RedAdd>(); return true; }
      return false;
  }
  return false;
}

// Internal reduce codes of thb200_var_dim / thb200_var_all (not part of the public enum).
enum { kRedVar = 100, kRedVarBiased = 101, kRedStd = 102, kRedStdBiased = 103 };
static int moments_code(int biased, int apply_sqrt) { return 100 + (biased ? 1 : 0) + (apply_sqrt ? 2 : 0); }

template <class F>
static bool dispatch_moments(int code, F&& f) {
  switch (code) {
    case kRedVar: f.template operator()<ModShift, RedMoments<false, false> >(); return true;
    case kRedVarBiased: f.template operator()<ModShift, RedMoments<true, false> >(); return true;
    case kRedStd: f.template operator()<ModShift, RedMoments<false, true> >(); return true;
    case kRedStdBiased: f.template operator()<ModShift, RedMoments<true, true> >(); return true;
  }
  return false;
}

template <class F>
static bool dispatch_red(int reduce, F&& f) {
  switch (reduce) {
    case THB200_RED_ADD: f.template operator()<RedAdd>(); return true;
    case THB200_RED_MUL: f.template operator()<RedMul>(); return true;
    case THB200_RED_MIN: f.template operator()<RedMin>(); return true;
    case THB200_RED_MAX: f.template operator()<RedMax>(); return true;
    case THB200_RED_AND: f.template operator()<RedAnd>(); return true;
    case THB200_RED_OR: f.template operator()<RedOr>(); return true;
  }
  return false;
}

template <class Red> struct IsMoments { static const bool value = false; };
template <bool B, bool S> struct IsMoments<RedMoments<B, S> > { static const bool value = true; };

struct ReduceAllArgs {
  cudaStream_t st;
  const thb200_tensor* in;
  int64_t n;
  float init, mparam;
  const float* mpoint;
  int fin;
  float fparam;
  float* d_out;
  float* scratch;
  bool contig;
  int head;
  Collapsed c;
  cudaError_t err = cudaSuccess;
  // cross-GPU exchange (thb200_exchange_push): cells the finishing block also stores the result to
  unsigned long long* const* push_cells = nullptr;
  int push_count = 0;
  unsigned int push_epoch = 0;
  bool pushed = false;

  template <class Red>
  void launch_pass2(int blocks) {
    if constexpr (IsMoments<Red>::value)
      thb_moments_all_pass2<Red><<<1, 1024, 0, st>>>((const ThbMoments*)scratch, blocks, fparam, d_out);
    else
      thb_reduce_all_pass2<Red><<<1, 1024, 0, st>>>((const typename Red::acc_t*)scratch, blocks, init, fin, fparam, d_out);
  }

  template <class Mod, class Red>
  void operator()() {
    const int blocks = (int)reduce_all_blocks(n);
    // one launch: the block that finishes last folds the partials (a separate pass 2 only if the
    // library's ticket counters cannot be addressed)
    ThbFinish F;
    F.ticket = reduce_ticket();
    F.fin = fin; F.fparam = fparam; F.out = d_out;
    F.push_cells = F.ticket ? push_cells : nullptr; F.push_count = push_count; F.push_epoch = push_epoch;
    pushed = F.push_cells != nullptr;
    if (contig) {
      const void* ptrs[1] = {in->data};
      stream_note_end(ptrs, 1, (size_t)n * sizeof(float), false);  // always walked upwards: the order of the additions is fixed
      // the kernel starts with a grid-dependency wait, so its blocks may be placed while the previous kernel drains
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)blocks);
      cfg.blockDim = dim3(THB_RA_THREADS);
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      cudaLaunchKernelEx(&cfg, thb_reduce_all_pass1_contig<Mod, Red>, (const float*)in->data, (thb_i64)n, head, init, mparam,
                         mpoint, (typename Red::acc_t*)scratch, F);
    } else {
      ThbLayout L;
      fill_layout(&L, in->data, c);
      thb_reduce_all_pass1_strided<Mod, Red><<<blocks, THB_RA_THREADS, 0, st>>>(
          L, (thb_u64)n, init, mparam, mpoint, (typename Red::acc_t*)scratch, F);
    }
    err = cudaGetLastError();
    if (err != cudaSuccess || F.ticket) return;
    launch_pass2<Red>(blocks);
    err = cudaGetLastError();
  }
};

// How many chunks the reduced dimension is cut into so that a reduction with few slices
// still fills the GPU: as many as fit one wave of resident blocks (`threads` worker threads
// per chunk in blocks of THB_RD_THREADS, `blocks_per_sm` of them resident), never a
// fraction of a wave more, and none when the slices alone fill half the GPU.
uint32_t pick_chunks(int64_t threads, int64_t rsize, int blocks_per_sm) {
  const int64_t wave = (int64_t)sm_count() * blocks_per_sm;
  const int64_t bx = (threads + THB_RD_THREADS - 1) / THB_RD_THREADS;
  if (bx * 2 > wave || rsize < 256) return 1;
  int64_t chunks = wave / bx;
  const int64_t max_chunks = rsize / 64;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks > 1024) chunks = 1024;
  if (chunks < 1) chunks = 1;
  // equal chunk lengths may need fewer chunks than asked for
  const int64_t len = (rsize + chunks - 1) / chunks;
  return (uint32_t)((rsize + len - 1) / len);
}
// resident blocks per SM of the column kernels (their __launch_bounds__)
static const int kOccSumV4 = RedAdd::kColsBlocks, kOccMomentsV4 = RedMoments<false, false>::kColsBlocks, kOccArgV4 = 4,
                 kOccScalar = 8;

// Whether 4 adjacent slices of a strided-dimension reduction are 4 consecutive, 16-byte
// aligned floats in every row: then one thread takes 4 slices with 128-bit loads.
static bool slices_vectorise(const float* data, const Collapsed& in_wo_rdim, int64_t rstride) {
  const int d = in_wo_rdim.dims;
  if (((uintptr_t)data & 15) != 0 || (rstride & 3) != 0) return false;
  if (in_wo_rdim.stride[d - 1] != 1 || (in_wo_rdim.size[d - 1] & 3) != 0) return false;
  for (int i = 0; i + 1 < d; ++i)
    if ((in_wo_rdim.stride[i] & 3) != 0) return false;
  return true;
}

// ---- TMA strip path (reduce_strip_kernels.cuh) -----------------------------------------
// max / min with indices: 4 consumer warps, one thread per column. Sums, products, variances:
// 8 consumer warps, two threads per column (even / odd rows), because their per-row work is a
// chain of fp64 conversions and additions that 4 warps per SM cannot hide.
// `t` as a row-major contiguous tensor split at `dim`: false if it is not one.
static bool contiguous_split(const thb200_tensor* t, int dim, int64_t* outer, int64_t* inner) {
  int64_t expect = 1;
  for (int d = t->ndim - 1; d >= 0; --d) {
    if (t->size[d] != 1 && t->stride[d] != expect) return false;
    expect *= t->size[d];
  }
  *outer = 1; *inner = 1;
  for (int d = 0; d < dim; ++d) *outer *= t->size[d];
  for (int d = dim + 1; d < t->ndim; ++d) *inner *= t->size[d];
  return true;
}

// Threads per column of the strip reductions with fp64 accumulators (4 measured the same as 2).
static const int kStripHalves = 2;

struct ReduceDimArgs {
  // strip path: contiguous [outer][rsize][inner] input, two partials per column and row chunk
  StripPlan strips;
  const float* src = nullptr;
  int64_t outer = 0, inner = 0;
  int strip_rc = 0;
  cudaStream_t st;
  ThbLayout out, in;
  uint32_t rsize, rstride, nslices;
  float init, mparam;
  float* scratch;
  uint32_t nchunks, chunk_len;
  bool vec4 = false;
  cudaError_t err = cudaSuccess;

  template <class Mod, class Red>
  void operator()() {
    const int sms = sm_count();
    if (rstride == 1) {
      if (rsize >= 8192) {
        unsigned blocks = nslices < (unsigned)kMaxGridBlocks ? nslices : (unsigned)kMaxGridBlocks;
        thb_reduce_dim_contig_block<Mod, Red><<<blocks, THB_RD_THREADS, 0, st>>>(out, in, rsize, nslices, init, mparam);
      } else {
        // a warp walks several short slices: measured faster than one block per 8 slices (0.86 against 0.81 of
        // the copy rate on 262144 slices of 1024)
        if (rsize <= 2048) {
          uint64_t blocks = ((uint64_t)nslices + 31) / 32;  // 8 lanes per slice
          if (blocks > (uint64_t)sms * 64) blocks = (uint64_t)sms * 64;
          thb_reduce_dim_contig_warp<Mod, Red, 8><<<(unsigned)blocks, THB_RD_THREADS, 0, st>>>(out, in, rsize, nslices, init, mparam);
        } else {
          uint64_t blocks = ((uint64_t)nslices + 7) / 8;
          if (blocks > (uint64_t)sms * 64) blocks = (uint64_t)sms * 64;
          thb_reduce_dim_contig_warp<Mod, Red, 32><<<(unsigned)blocks, THB_RD_THREADS, 0, st>>>(out, in, rsize, nslices, init, mparam);
        }
      }
      err = cudaGetLastError();
      return;
    }
    uint64_t bx = ((uint64_t)nslices + THB_RD_THREADS - 1) / THB_RD_THREADS;
    if (bx > 65535u * 16u) bx = 65535u * 16u;
    if (strips.ok) {
      typedef ThbReduceConsumer<Mod, Red> Cons;
      CUtensorMap map;
      strip_rc = make_strip_map(&map, src, outer, rsize, inner, inner);
      if (strip_rc) return;
      ThbStripGeom g;
      g.n = rsize; g.inner = inner; g.strips_per_outer = strips.strips_per_outer; g.total_strips = strips.total_strips;
      g.nchunks = strips.nchunks; g.chunk_rows = strips.chunk_rows; g.npartials = nchunks; g.nslices = nslices;
      typename Cons::Params cp;
      cp.out = out; cp.src = src; cp.partial = (typename Red::acc_t*)scratch; cp.init = init; cp.mparam = mparam;
      const int64_t items = (int64_t)strips.total_strips * strips.nchunks;
      const unsigned ctas = (unsigned)(items < sms ? items : sms);
      err = cudaFuncSetAttribute(thb_strip_reduce<Cons, kStripHalves>, cudaFuncAttributeMaxDynamicSharedMemorySize, THB_SS_SMEM);
      if (err != cudaSuccess) return;
      thb_strip_reduce<Cons, kStripHalves><<<ctas, 32 + 128 * kStripHalves, THB_SS_SMEM, st>>>(map, g, cp, device_status_word(STATUS_STRIP_REDUCE));
    } else if (vec4) {
      uint64_t bq = ((uint64_t)(nslices >> 2) + THB_RD_THREADS - 1) / THB_RD_THREADS;
      if (bq > 65535u * 16u) bq = 65535u * 16u;
      thb_reduce_dim_noncontig_v4<Mod, Red><<<dim3((unsigned)bq, nchunks), THB_RD_THREADS, 0, st>>>(
          out, in, rsize, rstride, nslices, chunk_len, nchunks, init, mparam, (typename Red::acc_t*)scratch);
    } else {
      thb_reduce_dim_noncontig<Mod, Red><<<dim3((unsigned)bx, nchunks), THB_RD_THREADS, 0, st>>>(
          out, in, rsize, rstride, nslices, chunk_len, nchunks, init, mparam, (typename Red::acc_t*)scratch);
    }
    err = cudaGetLastError();
    if (err != cudaSuccess || nchunks == 1) return;
    if (nchunks >= 8) {  // 32 slices x 8 chunk lanes per block
      uint64_t bf = ((uint64_t)nslices + 31) / 32;
      if (bf > 65535u * 16u) bf = 65535u * 16u;
      thb_reduce_dim_fold_chunks<Red, 8><<<(unsigned)bf, THB_RD_THREADS, 0, st>>>(
          out, (const typename Red::acc_t*)scratch, nslices, nchunks, init, rsize);
    } else {
      thb_reduce_dim_fold_chunks<Red, 1><<<(unsigned)bx, THB_RD_THREADS, 0, st>>>(
          out, (const typename Red::acc_t*)scratch, nslices, nchunks, init, rsize);
    }
    err = cudaGetLastError();
  }
};

struct FoldArgs {
  cudaStream_t st;
  const float* partials;
  int count;
  float init;
  float* d_out;
  cudaError_t err = cudaSuccess;
  template <class Red>
  void operator()() {
    thb_fold_floats<Red><<<1, 1024, 0, st>>>(partials, count, init, d_out);
    err = cudaGetLastError();
  }
};

static float identity_of(int reduce) {
  switch (reduce) {
    case THB200_RED_ADD: return 0.f;
    case THB200_RED_MUL: return 1.f;
    case THB200_RED_MIN: return __builtin_inff();
    case THB200_RED_MAX: return -__builtin_inff();
    case THB200_RED_AND: return 1.f;
    case THB200_RED_OR: return 0.f;
  }
  return 0.f;
}

template <bool IS_MAX>
static int argreduce(cudaStream_t st, float* values, float* indices, const float* src, int64_t outer, int64_t n,
                     int64_t inner, float* scratch, size_t scratch_bytes) {
  const int sms = sm_count();
  if (inner == 1) {
    if (n < 8192) {
      int64_t blocks = (outer + 7) / 8;
      if (blocks > kMaxGridBlocks) blocks = kMaxGridBlocks;
      thb_argreduce_rows<IS_MAX, true><<<(unsigned)blocks, THB_RD_THREADS, 0, st>>>(values, indices, src, outer, (thb_u32)n);
    } else {
      int64_t blocks = outer < kMaxGridBlocks ? outer : kMaxGridBlocks;
      thb_argreduce_rows<IS_MAX, false><<<(unsigned)blocks, THB_RD_THREADS, 0, st>>>(values, indices, src, outer, (thb_u32)n);
    }
    THB_CUDA(cudaGetLastError());
    return 0;
  }
  const int64_t nslices = outer * inner;
  const bool vec4 = (inner & 3) == 0 && ((uintptr_t)src & 15) == 0;
  const StripPlan sp = plan_strips(src, outer, n, inner);
  if (sp.ok) {
    typedef ThbArgConsumer<IS_MAX> Cons;
    const size_t need = sp.nchunks > 1 ? (size_t)sp.nchunks * nslices * 8 : 0;
    if (need && (!scratch || scratch_bytes < need))
      return fail("max/min: scratch too small (%zu bytes, need %zu)", scratch_bytes, need);
    CUtensorMap map;
    if (int rc = make_strip_map(&map, src, outer, n, inner, inner)) return rc;
    ThbStripGeom g;
    g.n = (thb_u32)n; g.inner = inner; g.strips_per_outer = sp.strips_per_outer; g.total_strips = sp.total_strips;
    g.nchunks = sp.nchunks; g.chunk_rows = sp.chunk_rows; g.npartials = sp.nchunks; g.nslices = (thb_u32)nslices;
    typename Cons::Params cp;
    cp.values = values; cp.indices = indices; cp.pval = scratch;
    cp.pidx = reinterpret_cast<int*>(scratch + (size_t)sp.nchunks * nslices);
    THB_CUDA(cudaFuncSetAttribute(thb_strip_reduce<Cons, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, THB_SS_SMEM));
    const int64_t items = (int64_t)sp.total_strips * sp.nchunks;
    const unsigned ctas = (unsigned)(items < sms ? items : sms);
    thb_strip_reduce<Cons, 1><<<ctas, THB_SS_THREADS, THB_SS_SMEM, st>>>(map, g, cp, device_status_word(STATUS_STRIP_ARGREDUCE));
    THB_CUDA(cudaGetLastError());
    if (sp.nchunks > 1) {
      if (sp.nchunks >= 8) {
        int64_t bf = (nslices + 31) / 32;
        if (bf > 65535 * 16) bf = 65535 * 16;
        thb_argreduce_fold_chunks<IS_MAX, 8><<<(unsigned)bf, THB_RD_THREADS, 0, st>>>(values, indices, cp.pval, cp.pidx, nslices, sp.nchunks);
      } else {
        int64_t bx = (nslices + THB_RD_THREADS - 1) / THB_RD_THREADS;
        if (bx > 65535 * 16) bx = 65535 * 16;
        thb_argreduce_fold_chunks<IS_MAX, 1><<<(unsigned)bx, THB_RD_THREADS, 0, st>>>(values, indices, cp.pval, cp.pidx, nslices, sp.nchunks);
      }
      THB_CUDA(cudaGetLastError());
    }
    return 0;
  }
  const uint32_t nchunks = vec4 ? pick_chunks(nslices >> 2, n, kOccArgV4) : pick_chunks(nslices, n, kOccScalar);
  const uint32_t chunk_len = (uint32_t)((n + nchunks - 1) / nchunks);
  float* pval = scratch;
  int* pidx = reinterpret_cast<int*>(scratch + (size_t)nchunks * nslices);
  if (nchunks > 1 && (!scratch || scratch_bytes < (size_t)nchunks * nslices * 8))
    return fail("max/min: scratch too small (%zu bytes, need %zu)", scratch_bytes, (size_t)nchunks * nslices * 8);
  int64_t bx = (nslices + THB_RD_THREADS - 1) / THB_RD_THREADS;
  if (bx > 65535 * 16) bx = 65535 * 16;
  if (vec4) {
    int64_t bq = ((nslices >> 2) + THB_RD_THREADS - 1) / THB_RD_THREADS;
    if (bq > 65535 * 16) bq = 65535 * 16;
    thb_argreduce_cols_v4<IS_MAX><<<dim3((unsigned)bq, nchunks), THB_RD_THREADS, 0, st>>>(
        values, indices, src, outer, (thb_u32)n, inner, chunk_len, nchunks, pval, pidx);
  } else {
    thb_argreduce_cols<IS_MAX><<<dim3((unsigned)bx, nchunks), THB_RD_THREADS, 0, st>>>(
        values, indices, src, outer, (thb_u32)n, inner, chunk_len, nchunks, pval, pidx);
  }
  THB_CUDA(cudaGetLastError());
  if (nchunks > 1) {
    if (nchunks >= 8) {  // 32 slices x 8 chunk lanes per block
      int64_t bf = (nslices + 31) / 32;
      if (bf > 65535 * 16) bf = 65535 * 16;
      thb_argreduce_fold_chunks<IS_MAX, 8><<<(unsigned)bf, THB_RD_THREADS, 0, st>>>(values, indices, pval, pidx, nslices, nchunks);
    } else {
      thb_argreduce_fold_chunks<IS_MAX, 1><<<(unsigned)bx, THB_RD_THREADS, 0, st>>>(values, indices, pval, pidx, nslices, nchunks);
    }
    THB_CUDA(cudaGetLastError());
  }
  return 0;
}

}  // namespace thb

using namespace thb;

extern "C" {

// one partial per pass-1 block; sums keep theirs in double
size_t thb200_reduce_all_scratch_bytes(int64_t n) { return (size_t)reduce_all_blocks(n) * sizeof(double); }

}  // extern "C"

namespace thb {
int reduce_all_impl(void* stream, int modify, int reduce, const thb200_tensor* in, float init, float mod_param,
                    const float* mod_point, int fin, float fin_param, float* d_out, float* scratch, size_t scratch_bytes,
                    unsigned long long* const* push_cells, int push_count, unsigned int push_epoch) {
  if (!in || !d_out) return fail("reduceAll: null argument");
  if (in->ndim > THB200_MAX_DIMS) return fail("reduceAll: too many dimensions");
  ReduceAllArgs a;
  a.st = (cudaStream_t)stream;
  a.in = in;
  a.n = num_elements(*in);
  a.init = init; a.mparam = mod_param; a.mpoint = mod_point;
  a.fin = fin; a.fparam = fin_param;
  a.d_out = d_out; a.scratch = scratch;
  a.push_cells = push_cells; a.push_count = push_count; a.push_epoch = push_epoch;
  if (a.n > 0 && !in->data) return fail("reduceAll: input has no device memory");
  if (!scratch || scratch_bytes < thb200_reduce_all_scratch_bytes(a.n))
    return fail("reduceAll: scratch too small (%zu bytes, need %zu)", scratch_bytes, thb200_reduce_all_scratch_bytes(a.n));
  if (!collapse(in->ndim, in->size, in->stride, -1, &a.c)) return fail("reduceAll: bad layout");
  a.contig = a.n == 0 || (a.c.contiguous() && ((uintptr_t)in->data & 3) == 0);
  a.head = a.contig && a.n > 0 ? (int)(((16 - ((uintptr_t)in->data & 15)) & 15) >> 2) : 0;
  if (a.head > a.n) a.head = (int)a.n;
  if (!a.contig && !can_use_32bit(in->ndim, in->size, in->stride))
    return fail("reduceAll: non-contiguous tensor needs 64-bit index math: not implemented");
  if (!dispatch_pair(modify, reduce, a.mparam, a)) return fail("reduceAll: unsupported modify/reduce pair (%d, %d)", modify, reduce);
  if (a.err != cudaSuccess) return fail_cuda(a.err, "reduceAll launch");
  if (push_cells && !a.pushed) return fail("exchange: the library's ticket counters are not available on this device");
  return 0;
}
}  // namespace thb

extern "C" {

int thb200_reduce_all(void* stream, int modify, int reduce, const thb200_tensor* in, float init, float mod_param,
                      const float* mod_point, int fin, float fin_param, float* d_out, float* scratch,
                      size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_reduce_all");
  return reduce_all_impl(stream, modify, reduce, in, init, mod_param, mod_point, fin, fin_param, d_out, scratch, scratch_bytes,
                         nullptr, 0, 0);
}

int thb200_fold_partials(void* stream, int reduce, const float* d_partials, int count, float* d_out) {
  THB_TIMED(stream, "thb200_fold_partials");
  if (!d_partials || !d_out || count < 1 || count > 1024) return fail("fold_partials: bad arguments");
  FoldArgs a;
  a.st = (cudaStream_t)stream;
  a.partials = d_partials; a.count = count; a.init = identity_of(reduce); a.d_out = d_out;
  if (!dispatch_red(reduce, a)) return fail("fold_partials: unknown reduce op %d", reduce);
  if (a.err != cudaSuccess) return fail_cuda(a.err, "fold_partials launch");
  return 0;
}

}  // extern "C"

namespace thb {
struct ExchangeFoldArgs {
  cudaStream_t st;
  const unsigned long long* cells;
  int count;
  unsigned int epoch;
  float init;
  float* d_out;
  unsigned long long limit_ns;
  int* status;
  cudaError_t err = cudaSuccess;
  template <class Red>
  void operator()() {
    // a programmatic dependent of the reduction before it: the block is resident and watching the cells
    // when the last of them arrives (the kernel waits for that reduction to complete before it writes)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    err = cudaLaunchKernelEx(&cfg, thb_exchange_wait_fold<Red>, cells, count, epoch, init, d_out, limit_ns, status);
    if (err == cudaSuccess) err = cudaGetLastError();
  }
};
int exchange_fold_launch(void* stream, int reduce, const unsigned long long* cells, int count, unsigned int epoch,
                         float* d_out, unsigned long long limit_ns) {
  ExchangeFoldArgs a;
  a.st = (cudaStream_t)stream;
  a.cells = cells; a.count = count; a.epoch = epoch; a.init = identity_of(reduce); a.d_out = d_out;
  a.limit_ns = limit_ns; a.status = device_status_word(STATUS_EXCHANGE);
  if (!a.status) return fail("exchange: the status word is not available");
  if (!dispatch_red(reduce, a)) return fail("exchange: unknown reduce op %d", reduce);
  if (a.err != cudaSuccess) return fail_cuda(a.err, "exchange fold launch");
  return 0;
}
float exchange_identity(int reduce) { return identity_of(reduce); }
}  // namespace thb

extern "C" {

static int reduce_dim_geometry(const thb200_tensor* in, int dim, int64_t* nslices, int64_t* rsize, int64_t* rstride) {
  if (!in || in->ndim < 1 || in->ndim > THB200_MAX_DIMS) return fail("reduceDim: bad input tensor");
  if (dim < 0 || dim >= in->ndim) return fail("reduceDim: dimension %d out of range", dim);
  *rsize = in->size[dim];
  *rstride = in->stride[dim];
  int64_t n = num_elements(*in);
  *nslices = *rsize > 0 ? n / *rsize : 0;
  return 0;
}

static size_t reduce_dim_scratch(const thb200_tensor* in, int dim, int occ_v4, size_t acc_bytes) {
  int64_t nslices, rsize, rstride;
  if (reduce_dim_geometry(in, dim, &nslices, &rsize, &rstride)) return 0;
  if (rstride == 1 || nslices == 0) return 0;
  Collapsed ci;
  if (!collapse(in->ndim, in->size, in->stride, dim, &ci)) return 0;
  int64_t outer, inner;
  if (contiguous_split(in, dim, &outer, &inner)) {
    const StripPlan sp = plan_strips(in->data, outer, rsize, inner);
    if (sp.ok) return (size_t)kStripHalves * sp.nchunks * nslices * acc_bytes;  // one partial per thread of a column and chunk
  }
  const bool vec4 = slices_vectorise(in->data, ci, rstride);
  uint32_t chunks = vec4 ? pick_chunks(nslices >> 2, rsize, occ_v4) : pick_chunks(nslices, rsize, kOccScalar);
  return chunks > 1 ? (size_t)chunks * nslices * acc_bytes : 0;
}

size_t thb200_reduce_dim_scratch_bytes(const thb200_tensor* in, int dim) {
  return reduce_dim_scratch(in, dim, kOccSumV4, sizeof(double));
}

// `reduce` is a THB200_RED_* code or one of the internal moments codes; `acc_bytes` the size
// of one chunk partial (8 for every public operator, 16 for the moments).
static int reduce_dim_impl(void* stream, int modify, int reduce, const thb200_tensor* out, const thb200_tensor* in,
                           int dim, float init, float mod_param, float* scratch, size_t scratch_bytes, size_t acc_bytes) {
  int64_t nslices, rsize, rstride;
  if (int rc = reduce_dim_geometry(in, dim, &nslices, &rsize, &rstride)) return rc;
  if (!out) return fail("reduceDim: null output");
  if (nslices == 0) return 0;
  if (num_elements(*out) != nslices) return fail("reduceDim: output has %lld elements, expected %lld",
                                                 (long long)num_elements(*out), (long long)nslices);
  if (!in->data || !out->data) return fail("reduceDim: tensor has no device memory");
  if (!can_use_32bit(in->ndim, in->size, in->stride) || !can_use_32bit(out->ndim, out->size, out->stride))
    return fail("reduceDim: tensor needs 64-bit index math: not implemented");
  Collapsed co, ci;
  if (!collapse(out->ndim, out->size, out->stride, -1, &co) || !collapse(in->ndim, in->size, in->stride, dim, &ci))
    return fail("reduceDim: bad layout");
  ReduceDimArgs a;
  a.st = (cudaStream_t)stream;
  fill_layout(&a.out, out->data, co);
  fill_layout(&a.in, in->data, ci);
  a.rsize = (uint32_t)rsize; a.rstride = (uint32_t)rstride; a.nslices = (uint32_t)nslices;
  a.init = init; a.mparam = mod_param; a.scratch = scratch;
  a.vec4 = rstride != 1 && slices_vectorise(in->data, ci, rstride);
  const int occ_v4 = reduce >= 100 ? kOccMomentsV4 : kOccSumV4;
  a.nchunks = rstride == 1 ? 1 : (a.vec4 ? pick_chunks(nslices >> 2, rsize, occ_v4) : pick_chunks(nslices, rsize, kOccScalar));
  a.chunk_len = (uint32_t)((rsize + a.nchunks - 1) / a.nchunks);
  if (rstride != 1 && contiguous_split(in, dim, &a.outer, &a.inner)) {
    a.strips = plan_strips(in->data, a.outer, rsize, a.inner);
    if (a.strips.ok) {
      a.src = in->data;
      a.nchunks = kStripHalves * a.strips.nchunks;  // partials to fold: one per thread of a column and chunk
    }
  }
  if (a.nchunks > 1 && (!scratch || scratch_bytes < (size_t)a.nchunks * nslices * acc_bytes))
    return fail("reduceDim: scratch too small (%zu bytes, need %zu)", scratch_bytes,
                (size_t)a.nchunks * nslices * acc_bytes);
  const bool known = reduce >= 100 ? dispatch_moments(reduce, a) : dispatch_pair(modify, reduce, mod_param, a);
  if (!known) return fail("reduceDim: unsupported modify/reduce pair (%d, %d)", modify, reduce);
  if (a.strip_rc) return a.strip_rc;
  if (a.err != cudaSuccess) return fail_cuda(a.err, "reduceDim launch");
  return 0;
}

int thb200_reduce_dim(void* stream, int modify, int reduce, const thb200_tensor* out, const thb200_tensor* in, int dim,
                      float init, float mod_param, float* scratch, size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_reduce_dim");
  if (reduce >= 100) return fail("reduceDim: unknown reduce op %d", reduce);
  return reduce_dim_impl(stream, modify, reduce, out, in, dim, init, mod_param, scratch, scratch_bytes, sizeof(double));
}

size_t thb200_var_dim_scratch_bytes(const thb200_tensor* in, int dim) {
  return reduce_dim_scratch(in, dim, kOccMomentsV4, sizeof(ThbMoments));
}

int thb200_var_dim(void* stream, const thb200_tensor* out, const thb200_tensor* in, int dim, int biased, int apply_sqrt,
                   float* scratch, size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_var_dim");
  return reduce_dim_impl(stream, THB200_MOD_COPY, moments_code(biased, apply_sqrt), out, in, dim, 0.f, 0.f, scratch,
                         scratch_bytes, sizeof(ThbMoments));
}

size_t thb200_var_all_scratch_bytes(int64_t n) { return (size_t)reduce_all_blocks(n) * sizeof(ThbMoments); }

int thb200_var_all(void* stream, const thb200_tensor* in, int biased, int apply_sqrt, float* d_out, float* scratch,
                   size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_var_all");
  if (!in || !d_out) return fail("varall: null argument");
  if (in->ndim > THB200_MAX_DIMS) return fail("varall: too many dimensions");
  ReduceAllArgs a;
  a.st = (cudaStream_t)stream;
  a.in = in;
  a.n = num_elements(*in);
  a.init = 0.f; a.mparam = 0.f;
  a.mpoint = a.n > 0 ? in->data : nullptr;  // the first element: the shift of ModShift
  a.fin = THB_FIN_NONE; a.fparam = (float)a.n;
  a.d_out = d_out; a.scratch = scratch;
  if (a.n > 0 && !in->data) return fail("varall: input has no device memory");
  if (!scratch || scratch_bytes < thb200_var_all_scratch_bytes(a.n))
    return fail("varall: scratch too small (%zu bytes, need %zu)", scratch_bytes, thb200_var_all_scratch_bytes(a.n));
  if (!collapse(in->ndim, in->size, in->stride, -1, &a.c)) return fail("varall: bad layout");
  a.contig = a.n == 0 || (a.c.contiguous() && ((uintptr_t)in->data & 3) == 0);
  a.head = a.contig && a.n > 0 ? (int)(((16 - ((uintptr_t)in->data & 15)) & 15) >> 2) : 0;
  if (a.head > a.n) a.head = (int)a.n;
  if (!a.contig && !can_use_32bit(in->ndim, in->size, in->stride))
    return fail("varall: non-contiguous tensor needs 64-bit index math: not implemented");
  dispatch_moments(moments_code(biased, apply_sqrt), a);
  if (a.err != cudaSuccess) return fail_cuda(a.err, "varall launch");
  return 0;
}

size_t thb200_reduce_dim_index_scratch_bytes(int64_t outer, int64_t n, int64_t inner) {
  if (inner <= 1 || outer * inner == 0) return 0;
  {
    // the strip path is taken when the source is 16-byte aligned, else the one-thread-per-column
    // kernels (128-bit variant: 4 slices per thread, hence more chunks): size for whichever needs more
    const StripPlan sp = plan_strips(nullptr, outer, n, inner);
    const size_t strips = (sp.ok && sp.nchunks > 1) ? (size_t)sp.nchunks * outer * inner * 8 : 0;
    uint32_t c = (inner & 3) == 0 ? pick_chunks((outer * inner) >> 2, n, kOccArgV4) : pick_chunks(outer * inner, n, kOccScalar);
    const size_t plain = c > 1 ? (size_t)c * outer * inner * 8 : 0;
    return strips > plain ? strips : plain;
  }
}

int thb200_reduce_dim_index(void* stream, int is_max, float* values, float* indices, const float* src, int64_t outer,
                            int64_t n, int64_t inner, float* scratch, size_t scratch_bytes) {
  THB_TIMED(stream, "thb200_reduce_dim_index");
  if (outer < 0 || n < 0 || inner < 0) return fail("max/min: negative extent");
  if (outer * inner == 0 || n == 0) return 0;
  if (!values || !indices || !src) return fail("max/min: null pointer");
  if (n >= (int64_t(1) << 24)) return fail("max/min: reduced dimension of %lld does not fit an fp32 index", (long long)n);
  if (n >= (int64_t(1) << 31)) return fail("max/min: dimension too large");
  return is_max ? argreduce<true>((cudaStream_t)stream, values, indices, src, outer, n, inner, scratch, scratch_bytes)
                : argreduce<false>((cudaStream_t)stream, values, indices, src, outer, n, inner, scratch, scratch_bytes);
}

}  // extern "C"

// ---- thb200_reduce_dim_noalloc ------------------------------------------------------
// Built-in scratch for callers that may not allocate device memory. It lives in the
// library's device image: every GPU that loads the library holds these 4 MiB until
// the process exits. In host code the array's name is only a handle for the runtime,
// not a device address: the address a kernel can use comes from cudaGetSymbolAddress,
// asked once per device with that device current.
// Status word of kernels with bounded waits (strip pipelines): lives in the device image like the
// built-in scratch below; its device address is looked up once per device.
static __device__ int thb_status_word_storage[thb::STATUS_FAMILIES];
static __device__ unsigned int thb_reduce_ticket_storage[64];

namespace thb {
// Set when a launch was given the status word of the device, cleared by thb200_kernel_status: a
// query with no such launch since the last one answers 0 without touching the GPU.
static std::atomic<bool> g_status_word_handed_out[64];

unsigned int* reduce_ticket() {
  static std::mutex mu;
  static unsigned int* base[64];
  static unsigned int next[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, thb_reduce_ticket_storage) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    base[dev] = (unsigned int*)p;
  }
  return base[dev] + (next[dev]++ & 63u);
}

int* device_status_word(int family) {
  static std::mutex mu;
  static int* addr[64];
  int dev = 0;
  if (family <= 0 || family >= STATUS_FAMILIES) return nullptr;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  g_status_word_handed_out[dev].store(true, std::memory_order_relaxed);
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, thb_status_word_storage) != cudaSuccess) return nullptr;
    addr[dev] = (int*)p;
  }
  return addr[dev] + family;
}

// Puts the 64 ticket counters of the current device back to zero (after a launch that may not
// have run to its end, a counter could otherwise stay non-zero and the next reduction that draws
// it would never write its result).
void reset_reduce_tickets(cudaStream_t st) {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, thb_reduce_ticket_storage) == cudaSuccess) cudaMemsetAsync(p, 0, sizeof(unsigned int) * 64, st);
  else cudaGetLastError();
}
}  // namespace thb

// One warp waits on a shared-memory barrier that nothing ever arrives on, with the given limit;
// when the wait gives up it stores `code` in the self-test status word, exactly as the pipelines do.
static __global__ void thb_selftest_wait_kernel(unsigned long long limit_ns, int code, int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    thb_mbar_init(thb_smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!thb_mbar_wait_ns(thb_smem_u32(&bar), 0, &abort_flag, limit_ns)) {
      abort_flag = 1;
      atomicCAS(status, 0, code);
    }
  }
  __syncthreads();
}

extern "C" int thb200_selftest_wait_expiry(void* stream, uint64_t limit_ns, int code) {
  if (limit_ns == 0 || limit_ns > 1000000000ull) return thb::fail("selftest: the limit must be between 1 ns and 1 s");
  if (code <= 0 || code > 255) return thb::fail("selftest: the code must be between 1 and 255");
  int* w = thb::device_status_word(thb::STATUS_SELFTEST);
  if (!w) return thb::fail("selftest: the status word is not available");
  thb_selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_ns, code, w);
  THB_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int thb200_kernel_status(void* stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 &&
      !thb::g_status_word_handed_out[dev].exchange(false, std::memory_order_relaxed))
    return 0;  // no kernel with bounded waits was launched since the last query
  int* w = thb::device_status_word(1);
  if (!w) { thb::fail("kernel_status: the status word is not available"); return -1; }
  w -= 1;  // the whole array
  if (dev >= 0 && dev < 64) thb::g_status_word_handed_out[dev].store(false, std::memory_order_relaxed);
  int h[thb::STATUS_FAMILIES];
  if (cudaMemcpyAsync(h, w, sizeof h, cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess ||
      cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) {
    thb::fail("kernel_status: could not read the status words");
    return -1;
  }
  int first = 0;
  for (int f = 1; f < thb::STATUS_FAMILIES; ++f)
    if (h[f] != 0 && first == 0) first = f * 256 + (h[f] & 255);
  if (first != 0) {
    cudaMemsetAsync(w, 0, sizeof h, (cudaStream_t)stream);
    // a kernel that gave up may have left its reduction ticket counter non-zero
    thb::reset_reduce_tickets((cudaStream_t)stream);
  }
  return first;
}

#define THB_NOALLOC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char thb_noalloc_scratch[THB_NOALLOC_SCRATCH_BYTES];

namespace thb {
static std::mutex g_noalloc_mu;
static void* g_noalloc_addr[64];  // per device ordinal; nullptr until the first call on that device
}  // namespace thb

extern "C" {

size_t thb200_reduce_dim_noalloc_capacity(void) { return THB_NOALLOC_SCRATCH_BYTES; }

int thb200_reduce_dim_noalloc(void* stream, int modify, int reduce, const thb200_tensor* out, const thb200_tensor* in,
                              int dim, float init, float mod_param) {
  const size_t need = thb200_reduce_dim_scratch_bytes(in, dim);
  if (need > THB_NOALLOC_SCRATCH_BYTES)
    return fail("reduceDim (no-alloc): this shape needs %zu bytes of scratch but the built-in scratch holds %u bytes; "
                "use thb200_reduce_dim with scratch of your own",
                need, (unsigned)THB_NOALLOC_SCRATCH_BYTES);
  int dev = 0;
  THB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail("reduceDim (no-alloc): device ordinal %d not supported", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_addr[dev]) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, thb_noalloc_scratch);
      if (e != cudaSuccess || !p) return fail_cuda(e, "cudaGetSymbolAddress(built-in scratch)");
      g_noalloc_addr[dev] = p;
    }
    scratch = g_noalloc_addr[dev];
  }
  // Nothing in the scratch has to start at zero: pass 1 writes every partial that pass 2 reads.
  return thb200_reduce_dim(stream, modify, reduce, out, in, dim, init, mod_param, (float*)scratch,
                           THB_NOALLOC_SCRATCH_BYTES);
}

}  // extern "C"
