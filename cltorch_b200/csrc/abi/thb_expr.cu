// User expressions for apply / map / map2: the x,y,z rewrite and the run-time
// compilation of the resulting operator body with NVRTC for sm_100a.
//
// The reference renders its OpenCL apply template with the operator string and
// compiles it on first use, caching by a key made of the operand count and the
// string (src/lib/THClApply.cpp:54-112). Here the text of apply_kernels.cuh is
// embedded in the library, the body becomes the `apply` member of a struct, and
// the five kernel templates are instantiated for it in one NVRTC program; the
// cubin is loaded through the CUDA runtime's library API and cached for the
// process by (operand count, body).
#include "thb_internal.h"
#include "../kernels/apply_kernels.cuh"

#include <nvrtc.h>
#include <cctype>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>

namespace thb {

static const char* kKernelSource =
#include "apply_kernels_src.inc"
    ;

// Function names whose accuracy policy differs from the CUDA fp32 routine
// (math_policy.cuh); expressions get the same policy as the built-in operators.
static const char* kPolicyMacros =
    "#define exp(x) thb_exp(x)\n"
    "#define tanh(x) thb_tanh(x)\n"
    "#define tan(x) thb_tan(x)\n"
    "#define sinh(x) thb_sinh(x)\n"
    "#define atan2(y, x) thb_atan2(y, x)\n"
    "#define pow(x, y) thb_pow(x, y)\n"
    "#define powr(x, y) thb_pow(x, y)\n"
    "#define pown(x, n) thb_pown(x, n)\n";

struct ExprEntry {
  ApplyKernels k;
  std::string body;
  std::string name;
  cudaLibrary_t lib = nullptr;
};

static std::mutex g_mu;
// key: device, operand count, body
static std::map<std::string, std::unique_ptr<ExprEntry>> g_cache;

static int fail_nvrtc(nvrtcResult r, const char* what, const std::string& log = "") {
  return fail("NVRTC error in %s: %s%s%s", what, nvrtcGetErrorString(r), log.empty() ? "" : "\n", log.c_str());
}

int expr_kernels(int nt, const std::string& body, const ApplyKernels** out) {
  if (nt < 1 || nt > 3) return fail("apply: %d tensors (1..3 supported)", nt);
  int dev = 0;
  THB_CUDA(cudaGetDevice(&dev));
  std::string key = std::to_string(dev) + "|" + std::to_string(nt) + "|" + body;
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) {
    *out = &it->second->k;
    return 0;
  }

  std::string src = kKernelSource;
  src += kPolicyMacros;
  src += "struct UserOp {\n  static constexpr bool kReadsOut = ";
  src += thb_body_reads_out(body.c_str()) ? "true" : "false";
  src += ";\n  static __device__ __forceinline__ void apply(float* out, const float* in1, const float* in2,\n"
         "      float val1, float val2, const float* pointTensor1, const float* pointTensor2) {\n    ";
  src += body;
  src += ";\n  }\n};\n";

  nvrtcProgram prog;
  nvrtcResult r = nvrtcCreateProgram(&prog, src.c_str(), "thb_user_expr.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) return fail_nvrtc(r, "nvrtcCreateProgram");
  const std::string nts = std::to_string(nt);
  const bool reads_out = thb_body_reads_out(body.c_str());
  const bool with_tma = nt >= 2 || reads_out;  // the TMA tile kernel needs at least one operand to load
  const int kMaxKernels = 6;
  const int kNumKernels = with_tma ? 6 : 5;
  const std::string names[kMaxKernels] = {
      "thb_apply_contig<UserOp, " + nts + ">", "thb_apply_strided<UserOp, " + nts + ">",
      "thb_apply_tile2d<UserOp, " + nts + ">", "thb_apply_rows2d<UserOp, " + nts + ">",
      "thb_apply_tile2d_v4<UserOp, " + nts + ">", "thb_apply_tile_tma<UserOp, " + nts + ">"};
  for (int i = 0; i < kNumKernels; ++i) {
    const std::string& n = names[i];
    r = nvrtcAddNameExpression(prog, n.c_str());
    if (r != NVRTC_SUCCESS) { nvrtcDestroyProgram(&prog); return fail_nvrtc(r, "nvrtcAddNameExpression"); }
  }
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false"};
  r = nvrtcCompileProgram(prog, 3, opts);
  if (r != NVRTC_SUCCESS) {
    size_t logn = 0;
    nvrtcGetProgramLogSize(prog, &logn);
    std::string log(logn, '\0');
    if (logn) nvrtcGetProgramLog(prog, &log[0]);
    nvrtcDestroyProgram(&prog);
    // keep the tail: the user's expression is at the end of the program
    if (log.size() > 800) log = log.substr(log.size() - 800);
    return fail("apply: expression did not compile: `%s`\n%s", body.c_str(), log.c_str());
  }
  size_t n = 0;
  r = nvrtcGetCUBINSize(prog, &n);
  if (r != NVRTC_SUCCESS || n == 0) { nvrtcDestroyProgram(&prog); return fail_nvrtc(r, "nvrtcGetCUBINSize"); }
  std::vector<char> cubin(n);
  r = nvrtcGetCUBIN(prog, cubin.data());
  if (r != NVRTC_SUCCESS) { nvrtcDestroyProgram(&prog); return fail_nvrtc(r, "nvrtcGetCUBIN"); }
  std::string lowered[kMaxKernels];
  for (int i = 0; i < kNumKernels; ++i) {
    const char* ln = nullptr;
    r = nvrtcGetLoweredName(prog, names[i].c_str(), &ln);
    if (r != NVRTC_SUCCESS || !ln) { nvrtcDestroyProgram(&prog); return fail_nvrtc(r, "nvrtcGetLoweredName"); }
    lowered[i] = ln;
  }
  nvrtcDestroyProgram(&prog);

  std::unique_ptr<ExprEntry> e(new ExprEntry);
  e->body = body;
  e->name = "expr";
  THB_CUDA(cudaLibraryLoadData(&e->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
  cudaKernel_t kern[kMaxKernels];
  for (int i = 0; i < kNumKernels; ++i) THB_CUDA(cudaLibraryGetKernel(&kern[i], e->lib, lowered[i].c_str()));
  e->k.contig = (const void*)kern[0];
  e->k.strided = (const void*)kern[1];
  e->k.tile2d = (const void*)kern[2];
  e->k.rows2d = (const void*)kern[3];
  e->k.tile2d_v4 = (const void*)kern[4];
  if (with_tma) e->k.tile_tma = (const void*)kern[5];
  e->k.nt = nt;
  e->k.reads_out = reads_out;
  e->k.name = e->name.c_str();
  e->k.body = e->body.c_str();
  *out = &e->k;
  g_cache[key] = std::move(e);
  return 0;
}

}  // namespace thb

extern "C" int thb200_rewrite_expr(const char* expr, int ntensors, char* out, size_t cap) {
  // Token-wise form of the reference's substring replacement
  // (src/lib/THClTensorMathPointwise.cpp:82-86,104-109,126-132): the identifiers
  // x, y, z become (*out), (*in1), (*in2); every other identifier (exp, max, ...)
  // is left alone. Floating literals without a suffix get `f` so that the
  // expression stays in fp32.
  if (!expr || !out) return -1;
  std::string r;
  const char* p = expr;
  while (*p) {
    unsigned char ch = (unsigned char)*p;
    if (isalpha(ch) || ch == '_') {
      const char* q = p;
      while (isalnum((unsigned char)*q) || *q == '_') ++q;
      std::string id(p, q);
      if (id == "x") r += "(*out)";
      else if (id == "y" && ntensors >= 2) r += "(*in1)";
      else if (id == "z" && ntensors >= 3) r += "(*in2)";
      else r += id;
      p = q;
    } else if (isdigit(ch) || (ch == '.' && isdigit((unsigned char)p[1]))) {
      const char* q = p;
      bool is_float = false;
      if (q[0] == '0' && (q[1] == 'x' || q[1] == 'X')) {
        q += 2;
        while (isxdigit((unsigned char)*q)) ++q;
      } else {
        while (isdigit((unsigned char)*q)) ++q;
        if (*q == '.') { is_float = true; ++q; while (isdigit((unsigned char)*q)) ++q; }
        if ((*q == 'e' || *q == 'E') && (isdigit((unsigned char)q[1]) || ((q[1] == '+' || q[1] == '-') && isdigit((unsigned char)q[2])))) {
          is_float = true;
          q += 2;
          while (isdigit((unsigned char)*q)) ++q;
        }
      }
      r.append(p, q);
      if (is_float) {
        if (*q == 'f' || *q == 'F' || *q == 'l' || *q == 'L') { r += 'f'; ++q; }
        else r += 'f';
      } else {
        while (*q == 'u' || *q == 'U' || *q == 'l' || *q == 'L') r += *q++;
      }
      p = q;
    } else {
      r += *p++;
    }
  }
  if (r.size() + 1 > cap) return -1;
  memcpy(out, r.c_str(), r.size() + 1);
  return (int)r.size();
}
