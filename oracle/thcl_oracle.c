/* thcl_oracle.c — CPU restatement of cltorch's apply / reduce / copy / BLAS path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA library: the
 * tests, the smoke check and the CPU-baseline leg of the benchmark call it; the
 * product never does. It follows the reference (hughperkins/cltorch, paths
 * relative to its root) function by function and is deliberately simple.
 *
 * Pinning: the reference cannot be built or run in this environment (no Lua /
 * Torch7, no OpenCL, EasyCL and clBLAS sources absent), and its own tests are
 * differential against Torch7 CPU tensors with almost no stored outputs. The
 * oracle is pinned against the known answers those tests do imply (literal
 * inputs with exactly representable results, and the formulas the tests spell
 * out in Lua), kept as fixtures under tests/golden/.
 *
 * Arithmetic: pointwise operators are evaluated in fp32 with one rounding per
 * operation (build with -ffp-contract=off), transcendental functions in double
 * rounded once to fp32; reductions and GEMM accumulate in double.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_MAX_DIMS 25 /* MAX_CLTORCH_DIMS, src/lib/THClReduceApplyUtils.h:19 */

typedef struct {
  float* data; /* element (0,...,0) of the view */
  int nd;
  const int64_t* size;
  const int64_t* stride;
} orc_tensor;

typedef struct {
  int dims;
  int64_t size[ORC_MAX_DIMS], stride[ORC_MAX_DIMS];
} orc_info;

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the timing loops; a launcher that exports OMP_NUM_THREADS=1 to every
 * rank would otherwise pin the CPU baseline to one core. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* TensorInfo<IndexType>::TensorInfo, src/lib/THClReduceApplyUtils.h:68-170. Written as the
 * reference writes it (two passes: count the collapsed dims, then fill), not as the
 * CUDA library does, so that the two are independent. */
int orc_collapse(int nd, const int64_t* size, const int64_t* stride, int reduce_dim, int64_t* out_size,
                 int64_t* out_stride) {
  int first = -1;
  for (int i = nd - 1; i >= 0; --i)
    if (size[i] != 1 && i != reduce_dim) { first = i; break; }
  if (first == -1) { out_size[0] = 1; out_stride[0] = 1; return 1; }
  int collapsed = nd - 1 - first;
  int64_t size_inner = size[first], stride_inner = stride[first];
  for (int i = first - 1; i >= 0; --i) {
    int64_t so = (i == reduce_dim) ? 1 : size[i], sto = stride[i];
    if (so == 1) { ++collapsed; continue; }
    if (sto == stride_inner * size_inner) { ++collapsed; size_inner *= so; continue; }
    size_inner = so; stride_inner = sto;
  }
  int dims = nd - collapsed;
  int idx = dims - 1;
  out_size[idx] = size[first];
  out_stride[idx] = stride[first];
  for (int i = first - 1; i >= 0; --i) {
    int64_t so = (i == reduce_dim) ? 1 : size[i], sto = stride[i];
    if (so == 1) continue;
    if (sto == out_size[idx] * out_stride[idx]) { out_size[idx] *= so; continue; }
    --idx;
    out_size[idx] = so;
    out_stride[idx] = sto;
  }
  return dims;
}

static void make_info(const orc_tensor* t, int reduce_dim, orc_info* o) {
  o->dims = orc_collapse(t->nd, t->size, t->stride, reduce_dim, o->size, o->stride);
}

/* IndexToOffset, src/lib/THClApply.cl:70-85 / src/lib/THClReduceApplyUtils.cl:26-65 */
static inline int64_t index_to_offset(const orc_info* o, int64_t lin) {
  int64_t off = 0;
  for (int d = o->dims - 1; d >= 0; --d) {
    off += (lin % o->size[d]) * o->stride[d];
    lin /= o->size[d];
  }
  return off;
}

int64_t orc_index_to_offset(int nd, const int64_t* size, const int64_t* stride, int64_t lin) {
  orc_info o;
  o.dims = orc_collapse(nd, size, stride, -1, o.size, o.stride);
  return index_to_offset(&o, lin);
}

static int64_t nelement(const orc_tensor* t) {
  if (t->nd <= 0) return 0;
  int64_t n = 1;
  for (int i = 0; i < t->nd; ++i) n *= t->size[i];
  return n;
}

/* THCL_overlappingIndices, src/lib/THClReduceApplyUtils.cpp:69-121 */
int orc_overlapping(int nd, const int64_t* size, const int64_t* stride) {
  int64_t s[ORC_MAX_DIMS], st[ORC_MAX_DIMS];
  int k = 0;
  for (int i = 0; i < nd; ++i)
    if (size[i] > 1) { s[k] = size[i]; st[k] = stride[i]; ++k; }
  if (k == 0) return 0;
  for (int i = 1; i < k; ++i) /* insertion sort by ascending stride */
    for (int j = i; j > 0 && st[j] < st[j - 1]; --j) {
      int64_t a = s[j]; s[j] = s[j - 1]; s[j - 1] = a;
      a = st[j]; st[j] = st[j - 1]; st[j - 1] = a;
    }
  if (st[0] < 1) return 1;
  for (int i = 1; i < k; ++i)
    if (st[i] < s[i - 1] * st[i - 1]) return 1;
  return 0;
}

/* ---- pointwise operators: the operator strings of the reference ------------- */
static inline float f_of_d(double x) { return (float)x; }
#define DBL1(fn, x) f_of_d(fn((double)(x)))

enum {
  OP_COPY_2, OP_FILL_1, OP_FILLPT_1, OP_ADDC_1, OP_ADDC_2, OP_MULC_1, OP_MULC_2, OP_ADDPT_1, OP_ADDPT_2, OP_SUBPT_1,
  OP_SUBPT_2, OP_MULPT_1, OP_MULPT_2, OP_DIVPT_1, OP_DIVPT_2, OP_ADD_2, OP_ADD_3, OP_CADD_2, OP_CADD_3, OP_SUB_2,
  OP_SUB_3, OP_CSUB_2, OP_CSUB_3, OP_MUL_2, OP_MUL_3, OP_CPOW_2, OP_CPOW_3, OP_DIV_2, OP_DIV_3, OP_ADDCMUL_3,
  OP_ADDCDIV_3, OP_CMAX_2, OP_CMAX_3, OP_CMIN_2, OP_CMIN_3, OP_CMAXV_1, OP_CMAXV_2, OP_CMINV_1, OP_CMINV_2,
  OP_SIGMOID, OP_POWN, OP_POW, OP_TPOW, OP_ATAN2_2, OP_ATAN2_3, OP_CLAMP, OP_SIGN, OP_LOG, OP_LOG1P, OP_EXP, OP_COS,
  OP_ACOS, OP_COSH, OP_SIN, OP_ASIN, OP_SINH, OP_TAN, OP_ATAN, OP_TANH, OP_SQRT, OP_CEIL, OP_FLOOR, OP_ABS, OP_ROUND,
  OP_NEG, OP_CINV, OP_LT, OP_GT, OP_LE, OP_GE, OP_EQ, OP_NE, OP_UNKNOWN
};

/* kinds of argument a family takes as its right-hand side */
enum { RHS_IN, RHS_VAL, RHS_PT };

typedef struct { int op; int nt; int rhs; } op_desc;

static int starts(const char* s, const char* p) { return strncmp(s, p, strlen(p)) == 0; }

/* Decodes the operator names of the CUDA library's table (NAME_<ntensors>, compare
 * families NAMEV_2 / NAMEPT_2 / NAMET_3). */
static op_desc decode(const char* name) {
  static const struct { const char* n; int op; } exact[] = {
      {"COPY_2", OP_COPY_2}, {"FILL_1", OP_FILL_1}, {"FILLPT_1", OP_FILLPT_1}, {"ADDC_1", OP_ADDC_1},
      {"ADDC_2", OP_ADDC_2}, {"MULC_1", OP_MULC_1}, {"MULC_2", OP_MULC_2}, {"ADDPT_1", OP_ADDPT_1},
      {"ADDPT_2", OP_ADDPT_2}, {"SUBPT_1", OP_SUBPT_1}, {"SUBPT_2", OP_SUBPT_2}, {"MULPT_1", OP_MULPT_1},
      {"MULPT_2", OP_MULPT_2}, {"DIVPT_1", OP_DIVPT_1}, {"DIVPT_2", OP_DIVPT_2}, {"ADD_2", OP_ADD_2},
      {"ADD_3", OP_ADD_3}, {"CADD_2", OP_CADD_2}, {"CADD_3", OP_CADD_3}, {"SUB_2", OP_SUB_2}, {"SUB_3", OP_SUB_3},
      {"CSUB_2", OP_CSUB_2}, {"CSUB_3", OP_CSUB_3}, {"MUL_2", OP_MUL_2}, {"MUL_3", OP_MUL_3}, {"CPOW_2", OP_CPOW_2},
      {"CPOW_3", OP_CPOW_3}, {"DIV_2", OP_DIV_2}, {"DIV_3", OP_DIV_3}, {"ADDCMUL_3", OP_ADDCMUL_3},
      {"ADDCDIV_3", OP_ADDCDIV_3}, {"CMAX_2", OP_CMAX_2}, {"CMAX_3", OP_CMAX_3}, {"CMIN_2", OP_CMIN_2},
      {"CMIN_3", OP_CMIN_3}, {"CMAXV_1", OP_CMAXV_1}, {"CMAXV_2", OP_CMAXV_2}, {"CMINV_1", OP_CMINV_1},
      {"CMINV_2", OP_CMINV_2}, {"ATAN2_2", OP_ATAN2_2}, {"ATAN2_3", OP_ATAN2_3}};
  static const struct { const char* n; int op; } unary[] = {
      {"SIGMOID", OP_SIGMOID}, {"POWN", OP_POWN}, {"POW", OP_POW}, {"TPOW", OP_TPOW}, {"CLAMP", OP_CLAMP},
      {"SIGN", OP_SIGN}, {"LOG1P", OP_LOG1P}, {"LOG", OP_LOG}, {"EXP", OP_EXP}, {"COSH", OP_COSH}, {"COS", OP_COS},
      {"ACOS", OP_ACOS}, {"SINH", OP_SINH}, {"SIN", OP_SIN}, {"ASIN", OP_ASIN}, {"TANH", OP_TANH}, {"TAN", OP_TAN},
      {"ATAN", OP_ATAN}, {"SQRT", OP_SQRT}, {"CEIL", OP_CEIL}, {"FLOOR", OP_FLOOR}, {"ABS", OP_ABS},
      {"ROUND", OP_ROUND}, {"NEG", OP_NEG}, {"CINV", OP_CINV}};
  static const struct { const char* n; int op; } cmp[] = {{"LT", OP_LT}, {"GT", OP_GT}, {"LE", OP_LE},
                                                           {"GE", OP_GE}, {"EQ", OP_EQ}, {"NE", OP_NE}};
  op_desc d = {OP_UNKNOWN, 0, RHS_IN};
  size_t len = strlen(name);
  if (len < 3) return d;
  for (size_t i = 0; i < sizeof exact / sizeof exact[0]; ++i)
    if (strcmp(name, exact[i].n) == 0) { d.op = exact[i].op; d.nt = name[len - 1] - '0'; return d; }
  for (size_t i = 0; i < sizeof unary / sizeof unary[0]; ++i) {
    size_t l = strlen(unary[i].n);
    if (len == l + 2 && starts(name, unary[i].n) && name[l] == '_') { d.op = unary[i].op; d.nt = name[len - 1] - '0'; return d; }
  }
  for (size_t i = 0; i < sizeof cmp / sizeof cmp[0]; ++i)
    if (starts(name, cmp[i].n)) {
      const char* r = name + 2;
      if (strcmp(r, "V_2") == 0) { d.op = cmp[i].op; d.nt = 2; d.rhs = RHS_VAL; return d; }
      if (strcmp(r, "PT_2") == 0) { d.op = cmp[i].op; d.nt = 2; d.rhs = RHS_PT; return d; }
      if (strcmp(r, "T_3") == 0) { d.op = cmp[i].op; d.nt = 3; d.rhs = RHS_IN; return d; }
    }
  return d;
}

static inline float unary_fn(int op, float x, float v1, float v2) {
  switch (op) {
    case OP_SIGMOID: return 1.0f / (1 + DBL1(exp, -x)); /* "1.0f / (1 + exp(- x))", src/lib/THClTensorMathPointwise.h:3-13 */
    case OP_POWN: return f_of_d(pow((double)x, (double)(int)v1));
    case OP_POW: return f_of_d(pow((double)x, (double)v1));
    case OP_TPOW: return f_of_d(pow((double)v1, (double)x));
    case OP_CLAMP: return fmaxf(fminf(x, v2), v1); /* src/lib/THClTensorMath2.cpp:113-131 */
    case OP_SIGN: return (float)((x > 0) - (x < 0));
    case OP_LOG: return DBL1(log, x);
    case OP_LOG1P: return DBL1(log1p, x);
    case OP_EXP: return DBL1(exp, x);
    case OP_COS: return DBL1(cos, x);
    case OP_ACOS: return DBL1(acos, x);
    case OP_COSH: return DBL1(cosh, x);
    case OP_SIN: return DBL1(sin, x);
    case OP_ASIN: return DBL1(asin, x);
    case OP_SINH: return DBL1(sinh, x);
    case OP_TAN: return DBL1(tan, x);
    case OP_ATAN: return DBL1(atan, x);
    case OP_TANH: return DBL1(tanh, x);
    case OP_SQRT: return sqrtf(x);
    case OP_CEIL: return ceilf(x);
    case OP_FLOOR: return floorf(x);
    case OP_ABS: return fabsf(x);
    case OP_ROUND: return roundf(x);
    case OP_NEG: return -x;
    case OP_CINV: return 1.0f / x;
  }
  return x;
}

static inline float compare_fn(int op, float a, float b) {
  switch (op) {
    case OP_LT: return a < b;
    case OP_GT: return a > b;
    case OP_LE: return a <= b;
    case OP_GE: return a >= b;
    case OP_EQ: return a == b;
    case OP_NE: return a != b;
  }
  return 0;
}

/* One element: *out, *in1, *in2, val1, val2, *pointTensor1 as in src/lib/THClApply.cl:33-45. */
static inline void op_element(op_desc d, float* out, const float* in1, const float* in2, float v1, float v2, float pt) {
  switch (d.op) {
    case OP_COPY_2: *out = *in1; break;
    case OP_FILL_1: *out = v1; break;
    case OP_FILLPT_1: *out = pt; break;
    case OP_ADDC_1: *out += v1; break;
    case OP_ADDC_2: *out = *in1 + v1; break;
    case OP_MULC_1: *out *= v1; break;
    case OP_MULC_2: *out = *in1 * v1; break;
    case OP_ADDPT_1: *out += pt; break;
    case OP_ADDPT_2: *out = *in1 + pt; break;
    case OP_SUBPT_1: *out -= pt; break;
    case OP_SUBPT_2: *out = *in1 - pt; break;
    case OP_MULPT_1: *out *= pt; break;
    case OP_MULPT_2: *out = *in1 * pt; break;
    case OP_DIVPT_1: *out /= pt; break;
    case OP_DIVPT_2: *out = *in1 / pt; break;
    case OP_ADD_2: *out += *in1; break;
    case OP_ADD_3: *out = *in1 + *in2; break;
    case OP_CADD_2: *out += v1 * *in1; break;
    case OP_CADD_3: *out = *in1 + v1 * *in2; break;
    case OP_SUB_2: *out -= *in1; break;
    case OP_SUB_3: *out = *in1 - *in2; break;
    case OP_CSUB_2: *out -= v1 * *in1; break;
    case OP_CSUB_3: *out = *in1 - v1 * *in2; break;
    case OP_MUL_2: *out *= *in1; break;
    case OP_MUL_3: *out = (*in1) * (*in2); break;
    case OP_CPOW_2: *out = f_of_d(pow((double)*out, (double)*in1)); break;
    case OP_CPOW_3: *out = f_of_d(pow((double)*in1, (double)*in2)); break;
    case OP_DIV_2: *out /= *in1; break;
    case OP_DIV_3: *out = *in1 / *in2; break;
    case OP_ADDCMUL_3: *out += v1 * *in1 * *in2; break; /* (val*in1)*in2, src/lib/THClTensorMath.cpp:177-192 */
    case OP_ADDCDIV_3: *out += v1 * *in1 / *in2; break;
    case OP_CMAX_2: *out = fmaxf(*out, *in1); break;
    case OP_CMAX_3: *out = fmaxf(*in1, *in2); break;
    case OP_CMIN_2: *out = fminf(*out, *in1); break;
    case OP_CMIN_3: *out = fminf(*in1, *in2); break;
    case OP_CMAXV_1: *out = fmaxf(*out, v1); break;
    case OP_CMAXV_2: *out = fmaxf(*in1, v1); break;
    case OP_CMINV_1: *out = fminf(*out, v1); break;
    case OP_CMINV_2: *out = fminf(*in1, v1); break;
    case OP_ATAN2_2: *out = f_of_d(atan2((double)*out, (double)*in1)); break;
    case OP_ATAN2_3: *out = f_of_d(atan2((double)*in1, (double)*in2)); break;
    case OP_LT: case OP_GT: case OP_LE: case OP_GE: case OP_EQ: case OP_NE:
      *out = compare_fn(d.op, *in1, d.rhs == RHS_VAL ? v1 : (d.rhs == RHS_PT ? pt : *in2));
      break;
    default:
      *out = unary_fn(d.op, d.nt == 1 ? *out : *in1, v1, v2);
  }
}

/* THClTensor_pointwiseApply + kernel THClTensor_pointwiseApplyD
 * (src/lib/THClApply.cpp:145-240, src/lib/THClApply.cl:47-102): for every linear index,
 * each operand's offset comes from the index decomposed in that operand's own collapsed
 * shape; only the element counts must agree. Returns 0, or -1 unknown op, -2 count
 * mismatch, -3 arity mismatch. */
int orc_apply(const char* opname, int nt, const orc_tensor* t, float v1, float v2, float pt) {
  op_desc d = decode(opname);
  if (d.op == OP_UNKNOWN) return -1;
  if (d.nt != nt) return -3;
  int64_t n = nelement(&t[0]);
  for (int i = 1; i < nt; ++i)
    if (nelement(&t[i]) != n) return -2;
  orc_info info[3];
  for (int i = 0; i < nt; ++i) make_info(&t[i], -1, &info[i]);
#pragma omp parallel for schedule(static)
  for (int64_t lin = 0; lin < n; ++lin) {
    float* out = t[0].data + index_to_offset(&info[0], lin);
    const float* in1 = nt >= 2 ? t[1].data + index_to_offset(&info[1], lin) : out;
    const float* in2 = nt >= 3 ? t[2].data + index_to_offset(&info[2], lin) : out;
    op_element(d, out, in1, in2, v1, v2, pt);
  }
  return 0;
}

/* ---- reductions --------------------------------------------------------------- */
enum { MOD_COPY = 0, MOD_ABSPOW = 1, MOD_NEZERO = 2, MOD_SQDEV = 3 };
enum { RED_ADD = 0, RED_MUL = 1, RED_MIN = 2, RED_MAX = 3, RED_AND = 4, RED_OR = 5 };

static inline double modify(int mod, float x, float p, double m) {
  switch (mod) {
    case MOD_ABSPOW: return (double)f_of_d(pow(fabs((double)x), (double)p)); /* pow(fabs(x), p), src/lib/THClTensorMath2.cpp:336-346 */
    case MOD_NEZERO: return x != 0.0f;
    case MOD_SQDEV: return ((double)x - m) * ((double)x - m);
  }
  return x;
}
static inline double reduce2(int red, double a, double b) {
  switch (red) {
    case RED_ADD: return a + b;
    case RED_MUL: return a * b;
    case RED_MIN: return fmin(a, b);
    case RED_MAX: return fmax(a, b);
    case RED_AND: return (double)((int)a && (int)b);
    case RED_OR: return (double)((int)a || (int)b);
  }
  return a;
}

/* THClTensor_reduceAll, src/lib/THClReduceAll.cpp:276-316: r = init; r = reduce(r, modify(e)). */
double orc_reduce_all(int mod, int red, const orc_tensor* in, double init, float mod_param, double mod_point) {
  int64_t n = nelement(in);
  orc_info info;
  make_info(in, -1, &info);
  double r = init;
  for (int64_t lin = 0; lin < n; ++lin)
    r = reduce2(red, r, modify(mod, in->data[index_to_offset(&info, lin)], mod_param, mod_point));
  return r;
}

/* THClTensor_reduceDim, src/lib/THClReduce.cpp:215-302 with the per-slice loop of
 * src/lib/THClReduce.cl:30-63. `out` has the input's shape with size 1 at `dim`. */
int orc_reduce_dim(int mod, int red, const orc_tensor* out, const orc_tensor* in, int dim, double init, float mod_param) {
  if (dim < 0 || dim >= in->nd) return -1;
  int64_t rsize = in->size[dim], rstride = in->stride[dim];
  int64_t nslices = rsize ? nelement(in) / rsize : 0;
  orc_info oi, ii;
  make_info(out, -1, &oi);
  make_info(in, dim, &ii);
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < nslices; ++s) {
    const float* p = in->data + index_to_offset(&ii, s);
    double r = init;
    for (int64_t i = 0; i < rsize; ++i) r = reduce2(red, r, modify(mod, p[i * rstride], mod_param, 0.0));
    out->data[index_to_offset(&oi, s)] = (float)r;
  }
  return 0;
}

/* THClTensor_kernel_transformReduceOuterDimIndex, src/lib/THClTensorMathTransformReduce.cl:17-41,
 * on a contiguous [outer][n][inner] source: acc = (-/+FLT_MAX, -1); an element replaces acc
 * only when strictly greater (smaller); index is 1-based. */
void orc_reduce_dim_index(int is_max, float* values, float* indices, const float* src, int64_t outer, int64_t n,
                          int64_t inner) {
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < outer * inner; ++s) {
    int64_t o = s / inner, i = s % inner;
    const float* p = src + o * n * inner + i;
    float acc = is_max ? -3.402823466e+38f : 3.402823466e+38f;
    float idx = -1;
    for (int64_t c = 0; c < n; ++c) {
      float x = p[c * inner];
      if (is_max ? (x > acc) : (x < acc)) { acc = x; idx = (float)(c + 1); }
    }
    values[s] = acc;
    indices[s] = idx;
  }
}

/* THClTensor_kernel_varOuterDim / varInnermostDim + THClTensor_computeVar
 * (src/lib/THClTensorMath2.cl:5-108; host side src/lib/THClTensorMath2.cpp:293-333, commented out
 * in the reference) on a contiguous [outer][n][inner] source: per slice sum and sum of squares,
 * then flag ? sum2/n - mean^2 : sum2/(n-1) - n/(n-1)*mean^2, clamped at 0, optional sqrt.
 * Evaluated in double (the reference accumulates in fp32). */
void orc_var_dim(int flag, int apply_sqrt, float* tgt, const float* src, int64_t outer, int64_t n, int64_t inner) {
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < outer * inner; ++s) {
    int64_t o = s / inner, i = s % inner;
    const float* p = src + o * n * inner + i;
    /* computeVar's sum2/n - mean^2 (flag) or sum2/(n-1) - n/(n-1)*mean^2 equals the mean of the
     * squared deviations over n (flag) or n-1; that form is evaluated here, in two passes, because
     * it does not cancel when the mean is far from zero */
    double mean = 0;
    for (int64_t c = 0; c < n; ++c) mean += (double)p[c * inner];
    mean /= (double)n;
    double sum2 = 0;
    for (int64_t c = 0; c < n; ++c) {
      double d = (double)p[c * inner] - mean;
      sum2 += d * d;
    }
    sum2 /= flag ? (double)n : (double)n - 1;
    sum2 = sum2 < 0 ? 0 : sum2;
    tgt[s] = (float)(apply_sqrt ? sqrt(sum2) : sum2);
  }
}

/* THClTensor_kernel_scanOuterDim (src/lib/THClTensorMathScan.cl:27-50): inclusive scan along n of
 * a contiguous [outer][n][inner] tensor, acc = init; acc = op(acc, x); store. is_mul selects
 * TensorMulOp (cumprod, init 1) over TensorAddOp (cumsum, init 0), src/lib/THClTensorMathScan.cpp:144-156.
 * The running value is kept in double (the reference keeps fp32). */
void orc_scan(int is_mul, float* tgt, const float* src, int64_t outer, int64_t n, int64_t inner) {
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < outer * inner; ++s) {
    int64_t o = s / inner, i = s % inner;
    const float* p = src + o * n * inner + i;
    float* t = tgt + o * n * inner + i;
    double acc = is_mul ? 1.0 : 0.0;
    for (int64_t c = 0; c < n; ++c) {
      acc = is_mul ? acc * (double)p[c * inner] : acc + (double)p[c * inner];
      t[c * inner] = (float)acc;
    }
  }
}

/* THClTensor_kernel_renorm (src/lib/THClTensorMath2.cl:110-143) on a contiguous [rows][size]
 * matrix, in place: norm = (sum |x|^value)^(1/value); rows with norm > maxnorm are multiplied by
 * maxnorm / (norm + 1e-7). Sums in double. */
void orc_renorm_rows(float* data, int64_t rows, int64_t size, float value, float maxnorm) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    float* row = data + r * size;
    double acc = 0;
    for (int64_t i = 0; i < size; ++i) acc += pow(fabs((double)row[i]), (double)value);
    float norm = (float)pow((double)(float)acc, 1.0 / (double)value);
    if (norm > maxnorm) {
      float f = (float)((double)maxnorm / ((double)norm + 1e-7));
      for (int64_t i = 0; i < size; ++i) row[i] *= f;
    }
  }
}

/* THClTensor_dist (src/lib/THClTensorMath2.cpp:448-475): (sum |a - b|^value)^(1/value) over two
 * contiguous vectors; the difference is taken in fp32 as the functor does, the sum in double. */
double orc_dist(const float* a, const float* b, int64_t n, float value) {
  double acc = 0;
#pragma omp parallel for schedule(static) reduction(+ : acc)
  for (int64_t i = 0; i < n; ++i) acc += pow(fabs((double)(float)(a[i] - b[i])), (double)value);
  return pow(acc, 1.0 / (double)value);
}

/* r = beta * t + alpha * m1 * m2 (THClTensor_addmm, src/lib/THClTensorMathBlas.cpp:107-214) on 2-D
 * strided views, fp64 accumulation. Batched form: the same for every index of a leading dim. */
void orc_addmm(float* r, int64_t r_s0, int64_t r_s1, float beta, const float* t, int64_t t_s0, int64_t t_s1, float alpha,
               const float* m1, int64_t a_s0, int64_t a_s1, const float* m2, int64_t b_s0, int64_t b_s1, int64_t M,
               int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      double acc = 0.0;
      for (int64_t k = 0; k < K; ++k) acc += (double)m1[i * a_s0 + k * a_s1] * (double)m2[k * b_s0 + j * b_s1];
      double base = beta == 0.0f ? 0.0 : (double)beta * (double)t[i * t_s0 + j * t_s1];
      r[i * r_s0 + j * r_s1] = (float)(base + (double)alpha * acc);
    }
}

/* ---- fp32 variants for timing the CPU path (contiguous data, all cores) --------
 * The arithmetic of a Torch7 FloatTensor: fp32 element operations (two roundings for a*x+b,
 * -ffp-contract=off), sums accumulated in double (TH's accreal for float). The library is built on
 * one host and timed on another, so the inner loops are compiled once per instruction set
 * (target_clones: baseline, AVX2, AVX-512) and the loader picks the widest the running CPU has;
 * that stands in for -march=native. Each thread works on one contiguous range (the ranges also
 * decide which NUMA node first touches a page, see orc_time_touch). */
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define ORC_CLONES __attribute__((target_clones("default", "avx2", "avx512f"), noinline))
#else
#define ORC_CLONES __attribute__((noinline))
#endif

ORC_CLONES static void k_map2_sqrt(float* restrict x, const float* restrict y, const float* restrict z, int64_t n) {
  for (int64_t i = 0; i < n; ++i) x[i] = sqrtf(1000 * x[i] + y[i] * 10 + z[i] * z[i]);
}
ORC_CLONES static void k_axpb(float* restrict x, int64_t n, float a, float b) {
  for (int64_t i = 0; i < n; ++i) x[i] = x[i] * a + b;
}
ORC_CLONES static void k_sqrt(float* restrict x, int64_t n) {
  for (int64_t i = 0; i < n; ++i) x[i] = sqrtf(x[i]);
}
ORC_CLONES static void k_mulc(float* restrict x, int64_t n, float a) {
  for (int64_t i = 0; i < n; ++i) x[i] *= a;
}
/* 16 independent double accumulators so that the additions vectorise and pipeline; folded in a fixed order */
ORC_CLONES static double k_sum(const float* restrict x, int64_t n) {
  double acc[16] = {0};
  int64_t i = 0;
  for (; i + 16 <= n; i += 16)
    for (int k = 0; k < 16; ++k) acc[k] += (double)x[i + k];
  double total = 0.0;
  for (int k = 0; k < 16; ++k) total += acc[k];
  for (; i < n; ++i) total += (double)x[i];
  return total;
}

#define ORC_RANGE(n)                                                     \
  int64_t t_ = omp_get_thread_num(), T_ = omp_get_num_threads();         \
  int64_t lo = (n) / T_ * t_ + ((n) % T_ < t_ ? (n) % T_ : t_);          \
  int64_t len = (n) / T_ + (t_ < (n) % T_ ? 1 : 0)

/* writes zeros with the same thread-to-range mapping as the loops below, so that on a multi-socket
 * host every page is first touched (and placed) by the thread that will work on it */
void orc_time_touch(float* x, int64_t n) {
#pragma omp parallel
  { ORC_RANGE(n); for (int64_t i = 0; i < len; ++i) x[lo + i] = 0.0f; }
}
void orc_time_map2_sqrt(float* x, const float* y, const float* z, int64_t n) {
#pragma omp parallel
  { ORC_RANGE(n); k_map2_sqrt(x + lo, y + lo, z + lo, len); }
}
void orc_time_axpb(float* x, int64_t n, float a, float b) {
#pragma omp parallel
  { ORC_RANGE(n); k_axpb(x + lo, len, a, b); }
}
void orc_time_sqrt(float* x, int64_t n) {
#pragma omp parallel
  { ORC_RANGE(n); k_sqrt(x + lo, len); }
}
void orc_time_mulc(float* x, int64_t n, float a) {
#pragma omp parallel
  { ORC_RANGE(n); k_mulc(x + lo, len, a); }
}
double orc_time_sum(const float* x, int64_t n) {
  double total = 0.0;
#pragma omp parallel reduction(+ : total)
  { ORC_RANGE(n); total += k_sum(x + lo, len); }
  return total;
}
