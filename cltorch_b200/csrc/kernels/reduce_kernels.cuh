// Reduction kernels for sm_100a: whole-tensor reductions (two passes, fixed
// order, no atomics), reductions along one dimension, and max/min along one
// dimension with the position of the extreme value.
//
// They replace the OpenCL kernels THClTensor_reduceAll / Pass1 / Pass2
// (reference src/lib/THClReduceAll.cl:24-100), THClTensor_reduceContigDim /
// reduceNoncontigDim (src/lib/THClReduce.cl:30-111), reduceBlock
// (src/lib/THClReduceApplyUtils.cl:76-124) and
// THClTensor_kernel_transformReduce{Outer,Innermost}DimIndex
// (src/lib/THClTensorMathTransformReduce.cl:17-102).
#pragma once
#include "apply_kernels.cuh"

// ---- modify / reduce operators ---------------------------------------------
// modifyOp strings of the reference: CopyOp "*out = *in1"; NormFunctor
// "pow(fabs(*in1), p)"; PartialNotEqualFunctor "*in1 != 0"
// (src/lib/THClTensorMath2.cpp:336-356); the squared deviation is the
// square_functor of the commented varall (src/lib/THClTensorMath2.cpp:197-207).
// |d|^p as a term of a norm or a distance. These terms are summed over many elements and
// the sum is held to 1e-5 relative, so the general power is exp2(p * log2(d)) on the
// special-function unit (relative error about 1e-6 for the exponents and magnitudes norms
// are taken with), unlike in the pointwise pow operator: a double-precision pow per element
// (about a hundred fp64 instructions) would make these reductions compute-bound.
__device__ __forceinline__ float thb_abs_pow(float d, float p) {
  d = fabsf(d);
  if (p == 2.0f) return d * d;
  if (p == 1.0f) return d;
  if (p == 0.0f) return 1.0f;  // pow(x, 0) = 1, also for x = 0
  if (p == 3.0f) return d * d * d;
  if (p == 4.0f) return (d * d) * (d * d);
  return __powf(d, p);
}

// kFirst: the operator wants the first element of the slice as its third argument.
struct ModCopy { static constexpr bool kFirst = false; static __device__ __forceinline__ float apply(float x, float, float) { return x; } };
// General exponent (the host routes p = 1, 2, 3 to the operators below, so no comparison of p is left in
// the loop): |x|^p = 2^(p log2|x|) on the special-function unit. p == 0 gives 1 for every x, also for 0.
__device__ __forceinline__ float thb_abs_pow_general(float x, float p) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(p * __log2f(fabsf(x))));
  return p == 0.0f ? 1.0f : r;
}
struct ModAbsPow { static constexpr bool kFirst = false; static __device__ __forceinline__ float apply(float x, float p, float) { return thb_abs_pow_general(x, p); } };
// Whether the four terms of a 128-bit vector may be added in fp32 before they join the double-precision sum.
// Only for the general power, whose terms carry the special-function unit's relative error of about 1e-6
// anyway: it saves three of four fp32 -> fp64 conversions, which share that unit with log2 and exp2.
template <class Mod> struct ThbAddsVectorInFloat { static constexpr bool value = false; };
template <> struct ThbAddsVectorInFloat<ModAbsPow> { static constexpr bool value = true; };
// |x|^p for the exponents norms are usually taken with: the host picks these when p is 1, 2 or 3,
// so that the loop carries no comparison of p per element.
struct ModAbs { static constexpr bool kFirst = false; static __device__ __forceinline__ float apply(float x, float, float) { return fabsf(x); } };
struct ModSquare { static constexpr bool kFirst = false; static __device__ __forceinline__ float apply(float x, float, float) { return x * x; } };
struct ModAbsCube { static constexpr bool kFirst = false; static __device__ __forceinline__ float apply(float x, float, float) { x = fabsf(x); return x * x * x; } };
struct ModNeZero { static constexpr bool kFirst = false; static __device__ __forceinline__ float apply(float x, float, float) { return x != 0.0f; } };
struct ModSqDev { static constexpr bool kFirst = false; static __device__ __forceinline__ float apply(float x, float, float m) { return (x - m) * (x - m); } };
// Deviation from the first element of the slice: the single-pass variance accumulates the
// sums of (x - k) and (x - k)^2, which keeps them small when the mean is far from zero.
struct ModShift { static constexpr bool kFirst = true; static __device__ __forceinline__ float apply(float x, float, float k) { return x - k; } };
// reduceOp strings: TensorAddOp, TensorMulOp, MinOp (fmin), MaxOp (fmax)
// (src/lib/THClTensorMathPointwise.h:62-140), logicalall/any functors
// "(int)*in1 && (int)*in2" (src/lib/THClTensorMath.cpp:444-460).
//
// Sums and products are accumulated in double and rounded to fp32 once, at the
// very end: the reduction stays bound by HBM (one DADD per 4-byte element is a
// fraction of the fp64 rate) and the result is within 1e-5 relative of a
// double-precision evaluation even for zero-mean data, where an fp32 tree loses
// digits to cancellation. min/max/and/or are exact in fp32.
struct RedAdd {
  static constexpr int kColsBlocks = 6;  // resident blocks per SM of the 128-bit column kernel
  typedef double acc_t;
  static __device__ __forceinline__ double apply(double a, double b) { return a + b; }
  static __device__ __forceinline__ float result(double a, float) { return (float)a; }
};
struct RedMul {
  static constexpr int kColsBlocks = 6;  // resident blocks per SM of the 128-bit column kernel
  typedef double acc_t;
  static __device__ __forceinline__ double apply(double a, double b) { return a * b; }
  static __device__ __forceinline__ float result(double a, float) { return (float)a; }
};
struct RedMin {
  static constexpr int kColsBlocks = 6;  // resident blocks per SM of the 128-bit column kernel
  typedef float acc_t;
  static __device__ __forceinline__ float apply(float a, float b) { return fminf(a, b); }
  static __device__ __forceinline__ float result(float a, float) { return a; }
};
struct RedMax {
  static constexpr int kColsBlocks = 6;  // resident blocks per SM of the 128-bit column kernel
  typedef float acc_t;
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
  static __device__ __forceinline__ float result(float a, float) { return a; }
};
struct RedAnd {
  static constexpr int kColsBlocks = 6;  // resident blocks per SM of the 128-bit column kernel
  typedef float acc_t;
  static __device__ __forceinline__ float apply(float a, float b) { return (float)((int)a && (int)b); }
  static __device__ __forceinline__ float result(float a, float) { return a; }
};
struct RedOr {
  static constexpr int kColsBlocks = 6;  // resident blocks per SM of the 128-bit column kernel
  typedef float acc_t;
  static __device__ __forceinline__ float apply(float a, float b) { return (float)((int)a || (int)b); }
  static __device__ __forceinline__ float result(float a, float) { return a; }
};

// Sum and sum of squares of a slice in one pass, for the variance / standard deviation of
// THClTensor_computeVar (src/lib/THClTensorMath2.cl:5-23): BIASED divides by n, otherwise by
// n - 1; negative results of the subtraction are clamped to 0; SQRT gives the standard
// deviation. Both sums are kept in double, so the subtraction loses nothing that fp32
// inputs could show. An element enters as ThbMoments(x) = (x, x * x).
struct ThbMoments {
  double s, q;
  __device__ __forceinline__ ThbMoments() {}
  __device__ __forceinline__ ThbMoments(float x) : s((double)x), q((double)x * (double)x) {}
};
template <bool BIASED, bool SQRT>
struct RedMoments {
  static constexpr int kColsBlocks = 4;  // 16-byte accumulators: 64 registers per thread
  typedef ThbMoments acc_t;
  static __device__ __forceinline__ ThbMoments apply(ThbMoments a, ThbMoments b) {
    a.s += b.s;
    a.q += b.q;
    return a;
  }
  // n = number of elements of the slice
  static __device__ __forceinline__ float result(ThbMoments a, float n_f) {
    const double n = (double)n_f;
    const double mean = a.s / n;
    double v = BIASED ? a.q / n - mean * mean : a.q / (n - 1.0) - n / (n - 1.0) * mean * mean;
    v = v < 0.0 ? 0.0 : v;
    return (float)(SQRT ? sqrt(v) : v);
  }
};

__device__ __forceinline__ float thb_shfl_down(float v, int off) { return __shfl_down_sync(0xffffffffu, v, off); }
__device__ __forceinline__ double thb_shfl_down(double v, int off) { return __shfl_down_sync(0xffffffffu, v, off); }
__device__ __forceinline__ ThbMoments thb_shfl_down(ThbMoments v, int off) {
  v.s = __shfl_down_sync(0xffffffffu, v.s, off);
  v.q = __shfl_down_sync(0xffffffffu, v.q, off);
  return v;
}

#define THB_FULL_MASK 0xffffffffu

// Folds the values of the calling block's threads in a fixed order; the result
// is valid in thread 0. `smem` holds one float per warp.
template <class Red>
__device__ __forceinline__ typename Red::acc_t thb_block_fold(typename Red::acc_t v, typename Red::acc_t init,
                                                              typename Red::acc_t* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = Red::apply(v, thb_shfl_down(v, off));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < nwarps ? smem[lane] : init;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = Red::apply(v, thb_shfl_down(v, off));
  }
  return v;
}

// ---- reduceAll --------------------------------------------------------------
// 256 threads x 8 float4 loads in flight per thread, 4 blocks per SM (<= 64 registers):
// 128 KB of loads in flight per SM, and 592 = 4 x 148 blocks are one full wave on a B200.
// The block count is a constant so that the summation order never depends on the device.
#define THB_RA_THREADS 256
#define THB_RA_UNROLL 8
#define THB_RA_BLOCKS_PER_SM 4
#define THB_RA_MAX_BLOCKS 592

#define THB_FIN_NONE 0
#define THB_FIN_DIV 1
#define THB_FIN_DIV_SQRT 2

// The block that finishes last folds the partials of all blocks and writes the scalar, so that a
// whole-tensor reduction is one launch. `ticket` counts the finished blocks (zero before the
// launch; the last block puts it back to zero); ticket == nullptr: a separate pass 2 does the fold.
struct ThbFinish {
  unsigned int* ticket = nullptr;
  int fin = 0;         // THB_FIN_*, ignored by the moments reductions
  float fparam = 1.f;  // divisor of the finaliser; element count for the moments
  float* out = nullptr;
  // Cross-GPU exchange (null otherwise): the block that writes the scalar also stores
  // (epoch << 32 | bits of the scalar) into push_cells[0 .. push_count), one 8-byte cell in the
  // memory of every GPU of the group (this GPU's own cell included), with plain stores.
  unsigned long long* const* push_cells = nullptr;
  int push_count = 0;
  unsigned int push_epoch = 0;
};

// One 8-byte store / load at system scope: whole or not at all, also across NVLink.
__device__ __forceinline__ void thb_store_cell(unsigned long long* cell, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(cell), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long thb_load_cell(const unsigned long long* cell) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(cell) : "memory");
  return v;
}

__device__ __forceinline__ float thb_load_partial(const float* p) { return __ldcg(p); }
__device__ __forceinline__ double thb_load_partial(const double* p) { return __ldcg(p); }
__device__ __forceinline__ ThbMoments thb_load_partial(const ThbMoments* p) {
  ThbMoments m;
  m.s = __ldcg(&p->s);
  m.q = __ldcg(&p->q);
  return m;
}
template <class Red>
__device__ __forceinline__ float thb_finish_value(Red*, typename Red::acc_t r, int fin, float fparam) {
  typedef typename Red::acc_t acc_t;
  if (fin == THB_FIN_DIV) r = r / (acc_t)fparam;
  else if (fin == THB_FIN_DIV_SQRT) r = sqrt(r / (acc_t)fparam);
  return (float)r;
}
template <bool B, bool S>
__device__ __forceinline__ float thb_finish_value(RedMoments<B, S>*, ThbMoments r, int, float n) {
  return RedMoments<B, S>::result(r, n);
}

// Called by every thread of every block after the block's partial is in partials[blockIdx.x].
// The fold order is fixed (thread t takes partials t, t + blockDim.x, ...; then the block fold), so
// the result does not depend on which block happens to come last.
template <class Red>
__device__ __forceinline__ void thb_finish_last_block(const ThbFinish& F, const typename Red::acc_t* partials, float init,
                                                      typename Red::acc_t* smem) {
  typedef typename Red::acc_t acc_t;
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    __threadfence();  // this block's partial before its ticket
    is_last = atomicAdd(F.ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();  // every other block's partial after its ticket
  acc_t r = (acc_t)init;
  for (unsigned int i = threadIdx.x; i < gridDim.x; i += blockDim.x) r = Red::apply(r, thb_load_partial(partials + i));
  r = thb_block_fold<Red>(r, (acc_t)init, smem);
  if (threadIdx.x == 0) {
    const float value = thb_finish_value((Red*)nullptr, r, F.fin, F.fparam);
    F.out[0] = value;
    *F.ticket = 0;
    if (F.push_cells) {
      const unsigned long long cell = ((unsigned long long)F.push_epoch << 32) | (unsigned long long)__float_as_uint(value);
      for (int j = 0; j < F.push_count; ++j) thb_store_cell(F.push_cells[j], cell);
    }
  }
}

// Pass 1 over one contiguous run. `head` as in thb_apply_contig.
template <class Mod, class Red>
__global__ void __launch_bounds__(THB_RA_THREADS, THB_RA_BLOCKS_PER_SM)
thb_reduce_all_pass1_contig(const float* in, thb_i64 n, int head, float init, float mparam,
                            const float* mpoint, typename Red::acc_t* partials, ThbFinish F) {
  typedef typename Red::acc_t acc_t;
  __shared__ acc_t smem[32];
  // launched with programmatic stream serialisation: the previous kernel of the stream has to be complete
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float mp = mpoint ? *mpoint : 0.f;
  const thb_i64 nvec = (n - head) >> 2;
  const float4* in4 = reinterpret_cast<const float4*>(in + head);
  acc_t acc[4] = {(acc_t)init, (acc_t)init, (acc_t)init, (acc_t)init};

  // Grid-stride over 32 KB pieces (256 threads x 8 vectors): at any moment the grid streams
  // through one window of consecutive pieces. Measured on 8 GiB: 7.1 TB/s, against 6.6 TB/s
  // with the 8 vectors of a thread spread 2.4 MB apart and 5.7 TB/s with one contiguous
  // share per block.
  const thb_i64 step = (thb_i64)gridDim.x * (THB_RA_THREADS * THB_RA_UNROLL);
  for (thb_i64 base = (thb_i64)blockIdx.x * (THB_RA_THREADS * THB_RA_UNROLL) + threadIdx.x; base < nvec;
       base += step) {
    float4 v[THB_RA_UNROLL];
#pragma unroll
    for (int u = 0; u < THB_RA_UNROLL; ++u) {
      thb_i64 i = base + u * THB_RA_THREADS;
      if (i < nvec) v[u] = in4[i];
    }
#pragma unroll
    for (int u = 0; u < THB_RA_UNROLL; ++u) {
      thb_i64 i = base + u * THB_RA_THREADS;
      if (i < nvec) {
        if (ThbAddsVectorInFloat<Mod>::value) {
          const float t = (Mod::apply(v[u].x, mparam, mp) + Mod::apply(v[u].y, mparam, mp)) +
                          (Mod::apply(v[u].z, mparam, mp) + Mod::apply(v[u].w, mparam, mp));
          acc[u & 3] = Red::apply(acc[u & 3], t);
        } else {
          acc[0] = Red::apply(acc[0], Mod::apply(v[u].x, mparam, mp));
          acc[1] = Red::apply(acc[1], Mod::apply(v[u].y, mparam, mp));
          acc[2] = Red::apply(acc[2], Mod::apply(v[u].z, mparam, mp));
          acc[3] = Red::apply(acc[3], Mod::apply(v[u].w, mparam, mp));
        }
      }
    }
  }
  if (blockIdx.x == 0) {
    const thb_i64 tail0 = head + (nvec << 2);
    const int ntail = (int)(n - tail0);
    const int t = threadIdx.x;
    if (t < head) acc[0] = Red::apply(acc[0], Mod::apply(in[t], mparam, mp));
    else if (t - head < ntail) acc[0] = Red::apply(acc[0], Mod::apply(in[tail0 + (t - head)], mparam, mp));
  }
  acc_t r = Red::apply(Red::apply(acc[0], acc[1]), Red::apply(acc[2], acc[3]));
  r = thb_block_fold<Red>(r, (acc_t)init, smem);
  if (threadIdx.x == 0) partials[blockIdx.x] = r;
  if (F.ticket) thb_finish_last_block<Red>(F, partials, init, smem);
}

// Pass 1 over any strided layout (32-bit index math).
template <class Mod, class Red>
__global__ void __launch_bounds__(THB_RA_THREADS)
thb_reduce_all_pass1_strided(ThbLayout L, thb_u64 n, float init, float mparam, const float* mpoint,
                             typename Red::acc_t* partials, ThbFinish F) {
  typedef typename Red::acc_t acc_t;
  __shared__ acc_t smem[32];
  const float mp = mpoint ? *mpoint : 0.f;
  acc_t acc = (acc_t)init;
  const thb_u64 step = (thb_u64)gridDim.x * (THB_RA_THREADS * THB_RA_UNROLL);
  for (thb_u64 base = (thb_u64)blockIdx.x * (THB_RA_THREADS * THB_RA_UNROLL) + threadIdx.x; base < n;
       base += step) {
    float v[THB_RA_UNROLL];
#pragma unroll
    for (int u = 0; u < THB_RA_UNROLL; ++u) {
      thb_u64 i = base + (thb_u64)u * THB_RA_THREADS;
      if (i < n) v[u] = L.data[thb_offset(L, (thb_u32)i)];
    }
#pragma unroll
    for (int u = 0; u < THB_RA_UNROLL; ++u) {
      thb_u64 i = base + (thb_u64)u * THB_RA_THREADS;
      if (i < n) acc = Red::apply(acc, Mod::apply(v[u], mparam, mp));
    }
  }
  acc = thb_block_fold<Red>(acc, (acc_t)init, smem);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
  if (F.ticket) thb_finish_last_block<Red>(F, partials, init, smem);
}


// Pass 2: one block folds the pass-1 partials and writes the finished scalar.
template <class Red>
__global__ void __launch_bounds__(1024)
thb_reduce_all_pass2(const typename Red::acc_t* partials, int count, float init, int fin, float fparam, float* out) {
  typedef typename Red::acc_t acc_t;
  __shared__ acc_t smem[32];
  acc_t r = (acc_t)init;
  for (int i = threadIdx.x; i < count; i += blockDim.x) r = Red::apply(r, partials[i]);
  r = thb_block_fold<Red>(r, (acc_t)init, smem);
  if (threadIdx.x == 0) {
    if (fin == THB_FIN_DIV) r = r / (acc_t)fparam;
    else if (fin == THB_FIN_DIV_SQRT) r = sqrt(r / (acc_t)fparam);
    out[0] = (float)r;
  }
}

// Pass 2 of the whole-tensor variance / standard deviation from single-pass moments.
template <class Red>
__global__ void __launch_bounds__(1024)
thb_moments_all_pass2(const ThbMoments* partials, int count, float n, float* out) {
  __shared__ ThbMoments smem[32];
  ThbMoments r(0.f);
  for (int i = threadIdx.x; i < count; i += blockDim.x) r = Red::apply(r, partials[i]);
  r = thb_block_fold<Red>(r, ThbMoments(0.f), smem);
  if (threadIdx.x == 0) out[0] = Red::result(r, n);
}

// The same fold for fp32 inputs (per-GPU results that already are point tensors).
template <class Red>
__global__ void __launch_bounds__(1024)
thb_fold_floats(const float* values, int count, float init, float* out) {
  typedef typename Red::acc_t acc_t;
  __shared__ acc_t smem[32];
  acc_t r = (acc_t)init;
  for (int i = threadIdx.x; i < count; i += blockDim.x) r = Red::apply(r, (acc_t)values[i]);
  r = thb_block_fold<Red>(r, (acc_t)init, smem);
  if (threadIdx.x == 0) out[0] = (float)r;
}

// Consumer side of the cross-GPU exchange: thread i waits until cell i of THIS GPU's buffer carries
// the expected epoch (its peer's store has arrived), then the values are folded exactly as
// thb_fold_floats folds an array. The wait is bounded: when a cell does not arrive within limit_ns
// the kernel stores 1 + (index of the first missing rank, at most 254) in *status, writes NaN and ends.
template <class Red>
__global__ void __launch_bounds__(1024)
thb_exchange_wait_fold(const unsigned long long* cells, int count, unsigned int epoch, float init, float* out,
                       unsigned long long limit_ns, int* status) {
  typedef typename Red::acc_t acc_t;
  __shared__ acc_t smem[32];
  __shared__ int missing;
  if (threadIdx.x == 0) missing = 0x7fffffff;
  __syncthreads();
  acc_t r = (acc_t)init;
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    unsigned long long t0 = 0, v = thb_load_cell(cells + i);
    for (unsigned int spin = 1; (unsigned int)(v >> 32) != epoch; ++spin) {
      if (spin == 1) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
      if ((spin & 31u) == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (now - t0 > limit_ns) { atomicMin(&missing, i); break; }
      }
      v = thb_load_cell(cells + i);
    }
    r = Red::apply(r, (acc_t)__uint_as_float((unsigned int)v));
  }
  __syncthreads();
  r = thb_block_fold<Red>(r, (acc_t)init, smem);
  // Launched as a programmatic dependent, the block has been watching the cells while the kernel before it
  // (this GPU's own reduction) was still running: the result is written only after that kernel has completed,
  // like everything a later kernel of the stream does.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    if (missing != 0x7fffffff) {
      if (status) atomicCAS(status, 0, 1 + (missing < 254 ? missing : 254));
      out[0] = __int_as_float(0x7fc00000);
    } else {
      out[0] = (float)r;
    }
  }
}

// ---- reduce along one dimension --------------------------------------------
// Slice s of the input starts at in.data[thb_offset(in, s)] (the layout has the
// reduced dimension forced to size 1) and has `rsize` elements `rstride` apart;
// its result goes to out.data[thb_offset(out, s)].

// rstride == 1, one block per slice (long slices).
#define THB_RD_THREADS 256
template <class Mod, class Red>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_reduce_dim_contig_block(ThbLayout out, ThbLayout in, thb_u32 rsize, thb_u32 nslices, float init,
                            float mparam) {
  typedef typename Red::acc_t acc_t;
  const float fin_n = (float)rsize;
  __shared__ acc_t smem[32];
  for (thb_u32 s = blockIdx.x; s < nslices; s += gridDim.x) {
    const float* p = in.data + thb_offset(in, s);
    const float k0 = Mod::kFirst ? p[0] : 0.f;
    acc_t acc[4] = {(acc_t)init, (acc_t)init, (acc_t)init, (acc_t)init};
    if ((((thb_u64)p) & 15) == 0 && (rsize & 3) == 0) {
      const float4* p4 = reinterpret_cast<const float4*>(p);
      const thb_u32 nvec = rsize >> 2;
      for (thb_u32 i = threadIdx.x; i < nvec; i += THB_RD_THREADS * 4) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i + u * THB_RD_THREADS < nvec) v[u] = p4[i + u * THB_RD_THREADS];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i + u * THB_RD_THREADS < nvec) {
            acc[0] = Red::apply(acc[0], Mod::apply(v[u].x, mparam, k0));
            acc[1] = Red::apply(acc[1], Mod::apply(v[u].y, mparam, k0));
            acc[2] = Red::apply(acc[2], Mod::apply(v[u].z, mparam, k0));
            acc[3] = Red::apply(acc[3], Mod::apply(v[u].w, mparam, k0));
          }
      }
    } else {
      for (thb_u32 i = threadIdx.x; i < rsize; i += THB_RD_THREADS)
        acc[0] = Red::apply(acc[0], Mod::apply(p[i], mparam, k0));
    }
    acc_t r = Red::apply(Red::apply(acc[0], acc[1]), Red::apply(acc[2], acc[3]));
    r = thb_block_fold<Red>(r, (acc_t)init, smem);
    if (threadIdx.x == 0) out.data[thb_offset(out, s)] = Red::result(r, fin_n);
    __syncthreads();
  }
}

// rstride == 1, short slices: G adjacent lanes per slice (G = 32: a warp per slice; G = 8: four
// slices per warp, for slices so short that the shuffle tree of a whole warp would cost as much as
// the additions). A group reads 16 * G contiguous bytes per load.
template <class Mod, class Red, int G>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_reduce_dim_contig_warp(ThbLayout out, ThbLayout in, thb_u32 rsize, thb_u32 nslices, float init,
                           float mparam) {
  typedef typename Red::acc_t acc_t;
  const float fin_n = (float)rsize;
  const int lane = threadIdx.x & 31;
  const int sub = lane % G;
  const thb_u32 per_warp = 32 / G, per_block = (THB_RD_THREADS / 32) * per_warp;
  for (thb_u64 s0 = (thb_u64)blockIdx.x * per_block + (threadIdx.x >> 5) * per_warp; s0 < nslices;
       s0 += (thb_u64)gridDim.x * per_block) {
    const thb_u64 s64 = s0 + lane / G;
    const bool live = s64 < nslices;
    const thb_u32 s = (thb_u32)s64;
    acc_t acc[4] = {(acc_t)init, (acc_t)init, (acc_t)init, (acc_t)init};
    if (live) {
      const float* p = in.data + thb_offset(in, s);
      const float k0 = Mod::kFirst ? p[0] : 0.f;
      if ((((thb_u64)p) & 15) == 0 && (rsize & 3) == 0) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
        const thb_u32 nvec = rsize >> 2;
        for (thb_u32 i = sub; i < nvec; i += G * 4) {
          float4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i + u * G < nvec) v[u] = p4[i + u * G];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i + u * G < nvec) {
              acc[0] = Red::apply(acc[0], Mod::apply(v[u].x, mparam, k0));
              acc[1] = Red::apply(acc[1], Mod::apply(v[u].y, mparam, k0));
              acc[2] = Red::apply(acc[2], Mod::apply(v[u].z, mparam, k0));
              acc[3] = Red::apply(acc[3], Mod::apply(v[u].w, mparam, k0));
            }
        }
      } else {
        for (thb_u32 i = sub; i < rsize; i += G) acc[0] = Red::apply(acc[0], Mod::apply(p[i], mparam, k0));
      }
    }
    acc_t r = Red::apply(Red::apply(acc[0], acc[1]), Red::apply(acc[2], acc[3]));
#pragma unroll
    for (int off = G / 2; off > 0; off >>= 1) r = Red::apply(r, thb_shfl_down(r, off));  // lane sub < off reads sub + off < G
    if (sub == 0 && live) out.data[thb_offset(out, s)] = Red::result(r, fin_n);
  }
}

// rstride != 1: one thread per (slice, chunk of the reduced dimension); adjacent
// threads take adjacent slices, so the loads coalesce whenever adjacent slices
// are adjacent in memory. With nchunks == 1 the result goes straight to `out`,
// otherwise to partial[chunk * nslices + slice] for thb_reduce_dim_fold_chunks.
template <class Mod, class Red>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_reduce_dim_noncontig(ThbLayout out, ThbLayout in, thb_u32 rsize, thb_u32 rstride, thb_u32 nslices,
                         thb_u32 chunk_len, thb_u32 nchunks, float init, float mparam,
                         typename Red::acc_t* partial) {
  typedef typename Red::acc_t acc_t;
  const float fin_n = (float)rsize;
  const thb_u32 chunk = blockIdx.y;
  const thb_u32 r0 = chunk * chunk_len;
  const thb_u32 r1 = min(rsize, r0 + chunk_len);
  for (thb_u64 s64 = (thb_u64)blockIdx.x * THB_RD_THREADS + threadIdx.x; s64 < nslices;
       s64 += (thb_u64)gridDim.x * THB_RD_THREADS) {
    const thb_u32 s = (thb_u32)s64;
    const float* p = in.data + thb_offset(in, s);
    const float k0 = Mod::kFirst ? p[0] : 0.f;
    acc_t acc = (acc_t)init;
    thb_u32 r = r0;
    for (; r + 16 <= r1; r += 16) {
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = p[(thb_u64)(r + u) * rstride];
#pragma unroll
      for (int u = 0; u < 16; ++u) acc = Red::apply(acc, Mod::apply(v[u], mparam, k0));
    }
    for (; r < r1; ++r) acc = Red::apply(acc, Mod::apply(p[(thb_u64)r * rstride], mparam, k0));
    if (nchunks == 1) out.data[thb_offset(out, s)] = Red::result(acc, fin_n);
    else partial[(thb_u64)chunk * nslices + s] = acc;
  }
}

// The same with one thread per 4 adjacent slices (128-bit loads): for layouts in which
// slices 4k..4k+3 are 4 consecutive floats at a 16-byte aligned address in every row of
// the reduced dimension. 8 rows in flight per thread.
template <class Mod, class Red>
__global__ void __launch_bounds__(THB_RD_THREADS, Red::kColsBlocks)
thb_reduce_dim_noncontig_v4(ThbLayout out, ThbLayout in, thb_u32 rsize, thb_u32 rstride, thb_u32 nslices,
                            thb_u32 chunk_len, thb_u32 nchunks, float init, float mparam,
                            typename Red::acc_t* partial) {
  typedef typename Red::acc_t acc_t;
  const float fin_n = (float)rsize;
  const thb_u32 chunk = blockIdx.y;
  const thb_u32 r0 = chunk * chunk_len;
  const thb_u32 r1 = min(rsize, r0 + chunk_len);
  const thb_u32 nquads = nslices >> 2;
  for (thb_u64 q64 = (thb_u64)blockIdx.x * THB_RD_THREADS + threadIdx.x; q64 < nquads;
       q64 += (thb_u64)gridDim.x * THB_RD_THREADS) {
    const thb_u32 s = (thb_u32)q64 << 2;
    const float* p = in.data + thb_offset(in, s);
    const float4 kq = Mod::kFirst ? *reinterpret_cast<const float4*>(p) : make_float4(0.f, 0.f, 0.f, 0.f);
    acc_t acc[4] = {(acc_t)init, (acc_t)init, (acc_t)init, (acc_t)init};
    thb_u32 r = r0;
    for (; r + 8 <= r1; r += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const float4*>(p + (thb_u64)(r + u) * rstride);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        acc[0] = Red::apply(acc[0], Mod::apply(v[u].x, mparam, kq.x));
        acc[1] = Red::apply(acc[1], Mod::apply(v[u].y, mparam, kq.y));
        acc[2] = Red::apply(acc[2], Mod::apply(v[u].z, mparam, kq.z));
        acc[3] = Red::apply(acc[3], Mod::apply(v[u].w, mparam, kq.w));
      }
    }
    for (; r < r1; ++r) {
      const float4 v = *reinterpret_cast<const float4*>(p + (thb_u64)r * rstride);
      acc[0] = Red::apply(acc[0], Mod::apply(v.x, mparam, kq.x));
      acc[1] = Red::apply(acc[1], Mod::apply(v.y, mparam, kq.y));
      acc[2] = Red::apply(acc[2], Mod::apply(v.z, mparam, kq.z));
      acc[3] = Red::apply(acc[3], Mod::apply(v.w, mparam, kq.w));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (nchunks == 1) out.data[thb_offset(out, s + j)] = Red::result(acc[j], fin_n);
      else partial[(thb_u64)chunk * nslices + s + j] = acc[j];
    }
  }
}

// Folds the chunk partials of every slice in chunk order. A block is (256 / LANES) slices x
// LANES lanes; lane k folds the k-th run of consecutive chunks, then lane 0 folds the run
// results in order, so LANES times as many threads share the latency-bound walk over the
// chunks (LANES = 8 when there are many chunks, 1 for a handful).
template <class Red, int LANES>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_reduce_dim_fold_chunks(ThbLayout out, const typename Red::acc_t* partial, thb_u32 nslices, thb_u32 nchunks,
                           float init, thb_u32 rsize) {
  typedef typename Red::acc_t acc_t;
  const float fin_n = (float)rsize;
  constexpr int SL = THB_RD_THREADS / LANES;
  __shared__ acc_t runs[LANES][SL + 1];
  const int tx = threadIdx.x % SL, ty = threadIdx.x / SL;
  const thb_u32 per = (nchunks + LANES - 1) / LANES;
  const thb_u32 c0 = min(nchunks, ty * per), c1 = min(nchunks, c0 + per);
  for (thb_u64 s0 = (thb_u64)blockIdx.x * SL; s0 < nslices; s0 += (thb_u64)gridDim.x * SL) {
    const thb_u64 s = s0 + tx;
    acc_t acc = (acc_t)init;
    if (s < nslices) {
      thb_u32 c = c0;
      for (; c + 4 <= c1; c += 4) {
        acc_t v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = partial[(thb_u64)(c + u) * nslices + s];
#pragma unroll
        for (int u = 0; u < 4; ++u) acc = Red::apply(acc, v[u]);
      }
      for (; c < c1; ++c) acc = Red::apply(acc, partial[(thb_u64)c * nslices + s]);
    }
    if (LANES > 1) {
      runs[ty][tx] = acc;
      __syncthreads();
      if (ty == 0) {
#pragma unroll
        for (int k = 1; k < LANES; ++k) acc = Red::apply(acc, runs[k][tx]);
      }
    }
    if (ty == 0 && s < nslices) out.data[thb_offset(out, (thb_u32)s)] = Red::result(acc, fin_n);
    if (LANES > 1) __syncthreads();
  }
}

// ---- max / min along one dimension with the position -----------------------
// A candidate is (value, 0-based position or -1). `Better(a, b)`: a replaces b.
// Within a thread positions ascend and the comparison is strict, so the first
// occurrence wins and NaN never replaces the running value; across threads the
// lower position wins ties, which gives the same answer as one sequential scan.
template <bool IS_MAX>
struct ThbArg {
  static __device__ __forceinline__ float start() { return IS_MAX ? -3.402823466e+38f : 3.402823466e+38f; }
  static __device__ __forceinline__ bool strictly(float a, float b) { return IS_MAX ? a > b : a < b; }
  static __device__ __forceinline__ void take(float& v, int& i, float ov, int oi) {
    if (strictly(ov, v) || (ov == v && oi < i)) { v = ov; i = oi; }
  }
};

// src viewed as [rows][n] contiguous; one warp (n < 1024) or one block per row.
template <bool IS_MAX, bool WARP_PER_ROW>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_argreduce_rows(float* values, float* indices, const float* src, thb_i64 rows, thb_u32 n) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const thb_i64 rows_per_block = WARP_PER_ROW ? THB_RD_THREADS / 32 : 1;
  for (thb_i64 row0 = (thb_i64)blockIdx.x * rows_per_block; row0 < rows; row0 += (thb_i64)gridDim.x * rows_per_block) {
    const thb_i64 row = WARP_PER_ROW ? row0 + warp : row0;
    float v = ThbArg<IS_MAX>::start();
    int idx = -1;
    if (row < rows) {
      const float* p = src + row * (thb_i64)n;
      const int t = WARP_PER_ROW ? lane : threadIdx.x;
      const int nt = WARP_PER_ROW ? 32 : THB_RD_THREADS;
      if ((((thb_u64)p) & 15) == 0 && (n & 3) == 0) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
        const thb_u32 nvec = n >> 2;
        for (thb_u32 i = t; i < nvec; i += nt * 2) {
          float4 a = p4[i];
          float4 b = (i + nt < nvec) ? p4[i + nt] : a;
          if (ThbArg<IS_MAX>::strictly(a.x, v)) { v = a.x; idx = 4 * i; }
          if (ThbArg<IS_MAX>::strictly(a.y, v)) { v = a.y; idx = 4 * i + 1; }
          if (ThbArg<IS_MAX>::strictly(a.z, v)) { v = a.z; idx = 4 * i + 2; }
          if (ThbArg<IS_MAX>::strictly(a.w, v)) { v = a.w; idx = 4 * i + 3; }
          if (i + nt < nvec) {
            const thb_u32 j = i + nt;
            if (ThbArg<IS_MAX>::strictly(b.x, v)) { v = b.x; idx = 4 * j; }
            if (ThbArg<IS_MAX>::strictly(b.y, v)) { v = b.y; idx = 4 * j + 1; }
            if (ThbArg<IS_MAX>::strictly(b.z, v)) { v = b.z; idx = 4 * j + 2; }
            if (ThbArg<IS_MAX>::strictly(b.w, v)) { v = b.w; idx = 4 * j + 3; }
          }
        }
      } else {
        for (thb_u32 i = t; i < n; i += nt)
          if (ThbArg<IS_MAX>::strictly(p[i], v)) { v = p[i]; idx = i; }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      float ov = __shfl_down_sync(THB_FULL_MASK, v, off);
      int oi = __shfl_down_sync(THB_FULL_MASK, idx, off);
      // a real position is only ever recorded for a value strictly beyond the start
      // value, so a candidate without a position (-1) has nothing to offer
      if (oi >= 0) ThbArg<IS_MAX>::take(v, idx, ov, oi);
    }
    if (WARP_PER_ROW) {
      if (lane == 0 && row < rows) {
        values[row] = v;
        indices[row] = (float)(idx < 0 ? -1 : idx + 1);
      }
    } else {
      if (lane == 0) { sv[warp] = v; si[warp] = idx; }
      __syncthreads();
      if (warp == 0) {
        v = lane < THB_RD_THREADS / 32 ? sv[lane] : ThbArg<IS_MAX>::start();
        idx = lane < THB_RD_THREADS / 32 ? si[lane] : -1;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          float ov = __shfl_down_sync(THB_FULL_MASK, v, off);
          int oi = __shfl_down_sync(THB_FULL_MASK, idx, off);
          if (oi >= 0) ThbArg<IS_MAX>::take(v, idx, ov, oi);
        }
        if (lane == 0) {
          values[row] = v;
          indices[row] = (float)(idx < 0 ? -1 : idx + 1);
        }
      }
      __syncthreads();
    }
  }
}

// src viewed as [outer][n][inner] contiguous with inner > 1: one thread per
// (outer, inner, chunk of n). With nchunks == 1 results go to values/indices,
// otherwise to pval/pidx[chunk * (outer*inner) + slice] for thb_argreduce_fold_chunks.
template <bool IS_MAX>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_argreduce_cols(float* values, float* indices, const float* src, thb_i64 outer, thb_u32 n, thb_i64 inner,
                   thb_u32 chunk_len, thb_u32 nchunks, float* pval, int* pidx) {
  const thb_i64 nslices = outer * inner;
  const thb_u32 chunk = blockIdx.y;
  const thb_u32 r0 = chunk * chunk_len;
  const thb_u32 r1 = min(n, r0 + chunk_len);
  for (thb_i64 s = (thb_i64)blockIdx.x * THB_RD_THREADS + threadIdx.x; s < nslices;
       s += (thb_i64)gridDim.x * THB_RD_THREADS) {
    const thb_i64 o = s / inner, i = s - o * inner;
    const float* p = src + (o * n) * inner + i;
    float v = ThbArg<IS_MAX>::start();
    int idx = -1;
    thb_u32 r = r0;
    for (; r + 16 <= r1; r += 16) {
      float x[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) x[u] = p[(thb_i64)(r + u) * inner];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (ThbArg<IS_MAX>::strictly(x[u], v)) { v = x[u]; idx = r + u; }
    }
    for (; r < r1; ++r) {
      float x = p[(thb_i64)r * inner];
      if (ThbArg<IS_MAX>::strictly(x, v)) { v = x; idx = r; }
    }
    if (nchunks == 1) {
      values[s] = v;
      indices[s] = (float)(idx < 0 ? -1 : idx + 1);
    } else {
      pval[(thb_i64)chunk * nslices + s] = v;
      pidx[(thb_i64)chunk * nslices + s] = idx;
    }
  }
}

// The same with one thread per 4 adjacent inner positions (inner % 4 == 0, src 16-byte aligned).
template <bool IS_MAX>
__global__ void __launch_bounds__(THB_RD_THREADS, 4)
thb_argreduce_cols_v4(float* values, float* indices, const float* src, thb_i64 outer, thb_u32 n, thb_i64 inner,
                      thb_u32 chunk_len, thb_u32 nchunks, float* pval, int* pidx) {
  const thb_i64 nslices = outer * inner;
  const thb_i64 nquads = nslices >> 2;
  const thb_u32 chunk = blockIdx.y;
  const thb_u32 r0 = chunk * chunk_len;
  const thb_u32 r1 = min(n, r0 + chunk_len);
  for (thb_i64 q = (thb_i64)blockIdx.x * THB_RD_THREADS + threadIdx.x; q < nquads;
       q += (thb_i64)gridDim.x * THB_RD_THREADS) {
    const thb_i64 s = q << 2;
    const thb_i64 o = s / inner, i = s - o * inner;
    const float* p = src + (o * n) * inner + i;
    float v[4];
    int idx[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[j] = ThbArg<IS_MAX>::start(); idx[j] = -1; }
    thb_u32 r = r0;
    for (; r + 8 <= r1; r += 8) {
      float4 x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) x[u] = *reinterpret_cast<const float4*>(p + (thb_i64)(r + u) * inner);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (ThbArg<IS_MAX>::strictly(x[u].x, v[0])) { v[0] = x[u].x; idx[0] = r + u; }
        if (ThbArg<IS_MAX>::strictly(x[u].y, v[1])) { v[1] = x[u].y; idx[1] = r + u; }
        if (ThbArg<IS_MAX>::strictly(x[u].z, v[2])) { v[2] = x[u].z; idx[2] = r + u; }
        if (ThbArg<IS_MAX>::strictly(x[u].w, v[3])) { v[3] = x[u].w; idx[3] = r + u; }
      }
    }
    for (; r < r1; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(p + (thb_i64)r * inner);
      if (ThbArg<IS_MAX>::strictly(x.x, v[0])) { v[0] = x.x; idx[0] = r; }
      if (ThbArg<IS_MAX>::strictly(x.y, v[1])) { v[1] = x.y; idx[1] = r; }
      if (ThbArg<IS_MAX>::strictly(x.z, v[2])) { v[2] = x.z; idx[2] = r; }
      if (ThbArg<IS_MAX>::strictly(x.w, v[3])) { v[3] = x.w; idx[3] = r; }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (nchunks == 1) {
        values[s + j] = v[j];
        indices[s + j] = (float)(idx[j] < 0 ? -1 : idx[j] + 1);
      } else {
        pval[(thb_i64)chunk * nslices + s + j] = v[j];
        pidx[(thb_i64)chunk * nslices + s + j] = idx[j];
      }
    }
  }
}

// Chunk candidates of every slice, folded in chunk order with the strict comparison (an
// earlier chunk keeps a tie); lanes as in thb_reduce_dim_fold_chunks.
template <bool IS_MAX, int LANES>
__global__ void __launch_bounds__(THB_RD_THREADS)
thb_argreduce_fold_chunks(float* values, float* indices, const float* pval, const int* pidx, thb_i64 nslices,
                          thb_u32 nchunks) {
  constexpr int SL = THB_RD_THREADS / LANES;
  __shared__ float rv[LANES][SL + 1];
  __shared__ int ri[LANES][SL + 1];
  const int tx = threadIdx.x % SL, ty = threadIdx.x / SL;
  const thb_u32 per = (nchunks + LANES - 1) / LANES;
  const thb_u32 c0 = min(nchunks, ty * per), c1 = min(nchunks, c0 + per);
  for (thb_i64 s0 = (thb_i64)blockIdx.x * SL; s0 < nslices; s0 += (thb_i64)gridDim.x * SL) {
    const thb_i64 s = s0 + tx;
    float v = ThbArg<IS_MAX>::start();
    int idx = -1;
    if (s < nslices) {
      for (thb_u32 c = c0; c < c1; ++c) {
        const float ov = pval[(thb_i64)c * nslices + s];
        const int oi = pidx[(thb_i64)c * nslices + s];
        if (oi >= 0 && ThbArg<IS_MAX>::strictly(ov, v)) { v = ov; idx = oi; }
      }
    }
    if (LANES > 1) {
      rv[ty][tx] = v;
      ri[ty][tx] = idx;
      __syncthreads();
      if (ty == 0) {
#pragma unroll
        for (int k = 1; k < LANES; ++k)
          if (ri[k][tx] >= 0 && ThbArg<IS_MAX>::strictly(rv[k][tx], v)) { v = rv[k][tx]; idx = ri[k][tx]; }
      }
    }
    if (ty == 0 && s < nslices) {
      values[s] = v;
      indices[s] = (float)(idx < 0 ? -1 : idx + 1);
    }
    if (LANES > 1) __syncthreads();
  }
}
