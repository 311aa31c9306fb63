// User-written kernels compiled at run time: the NVRTC counterpart of torch.ClKernel
// (reference src/UserKernel.cpp:217-381). The caller names its arguments (tensors, ints,
// floats) and supplies the kernel body; the body sees every tensor `t` as
// `t_info` (sizes, strides, offset, dims: struct THClTensorInfoCl of
// src/lib/THClTensorInfoCl.cl) and `t_data` (start of the storage), exactly as the
// reference renders them (src/UserKernel.cpp:75-89, 256-272). A prelude maps the OpenCL C
// functions such kernels use (get_global_id, barrier ...) onto CUDA, and the address-space
// words (global, local) are rewritten in the user's text.
#include "thb_internal.h"

#include <nvrtc.h>

#include <cctype>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

struct thb200_user_kernel {
  std::string name, rendered;
  std::vector<int> kinds;
  cudaLibrary_t lib = nullptr;
  cudaKernel_t kernel = nullptr;
  int device = 0;
};

namespace thb {

struct TensorInfoCl {  // layout of struct THClTensorInfoCl
  unsigned int sizes[THB200_MAX_DIMS];
  unsigned int strides[THB200_MAX_DIMS];
  int offset;
  int dims;
};

static const char* kOpenClPrelude =
    "typedef struct THClTensorInfoCl {\n"
    "  unsigned int sizes[25];\n"
    "  unsigned int strides[25];\n"
    "  int offset;\n"
    "  int dims;\n"
    "} TensorInfoCl;\n"
    "#define get_global_id(d) ((d) == 0 ? (int)(blockIdx.x * blockDim.x + threadIdx.x) : 0)\n"
    "#define get_local_id(d) ((d) == 0 ? (int)threadIdx.x : 0)\n"
    "#define get_group_id(d) ((d) == 0 ? (int)blockIdx.x : 0)\n"
    "#define get_local_size(d) ((d) == 0 ? (int)blockDim.x : 1)\n"
    "#define get_num_groups(d) ((d) == 0 ? (int)gridDim.x : 1)\n"
    "#define get_global_size(d) ((d) == 0 ? (int)(gridDim.x * blockDim.x) : 1)\n"
    "#define CLK_LOCAL_MEM_FENCE 1\n"
    "#define CLK_GLOBAL_MEM_FENCE 2\n"
    "#define barrier(flags) __syncthreads()\n"
    "#define thb_mem_fence(flags) __threadfence_block()\n"
    "#define mad(a, b, c) ((a) * (b) + (c))\n";

// The OpenCL address-space words cannot be macros (CUDA's own __global__ / __shared__ expand
// to attributes spelt with the same identifiers), so they are replaced token by token in the
// user's text: global, __global, constant-free pointers -> nothing; local, __local ->
// __shared__. Comments and string literals are copied as they are.
static std::string translate_opencl_words(const std::string& in) {
  std::string out;
  size_t i = 0;
  const size_t n = in.size();
  while (i < n) {
    const char c = in[i];
    if (c == '/' && i + 1 < n && in[i + 1] == '/') {
      const size_t e = in.find('\n', i);
      out.append(in, i, e == std::string::npos ? n - i : e - i);
      i = e == std::string::npos ? n : e;
    } else if (c == '/' && i + 1 < n && in[i + 1] == '*') {
      size_t e = in.find("*/", i + 2);
      e = e == std::string::npos ? n : e + 2;
      out.append(in, i, e - i);
      i = e;
    } else if (c == '"' || c == '\'') {
      size_t e = i + 1;
      while (e < n && in[e] != c) e += (in[e] == '\\' && e + 1 < n) ? 2 : 1;
      e = e < n ? e + 1 : n;
      out.append(in, i, e - i);
      i = e;
    } else if (isalpha((unsigned char)c) || c == '_') {
      size_t e = i;
      while (e < n && (isalnum((unsigned char)in[e]) || in[e] == '_')) ++e;
      const std::string id = in.substr(i, e - i);
      if (id == "global" || id == "__global" || id == "kernel" || id == "__kernel") {
        out += "";
      } else if (id == "constant" || id == "__constant" || id == "local" || id == "__local") {
        // A declared object ("local float buf[64];", "constant float w[2] = {...};") becomes a
        // __shared__ / __constant__ object. Where the word qualifies a pointer ("float f(local float*
        // buf)", a '*' follows before the declaration ends) CUDA spells the pointer without it.
        size_t q = e;
        while (q < n && in[q] != '*' && in[q] != ';' && in[q] != ',' && in[q] != ')' && in[q] != '[' && in[q] != '=' && in[q] != '{') ++q;
        const bool pointer = q < n && in[q] == '*';
        if (id == "local" || id == "__local") out += pointer ? "" : "__shared__";
        else out += pointer ? "const" : "__constant__";
      } else if (id == "mem_fence" || id == "read_mem_fence" || id == "write_mem_fence") {
        out += "thb_mem_fence";
      } else {
        out += id;
      }
      i = e;
    } else if (isdigit((unsigned char)c)) {  // a number may contain letters (1e5f, 0x1F): copy it whole
      size_t e = i;
      while (e < n && (isalnum((unsigned char)in[e]) || in[e] == '.')) ++e;
      out.append(in, i, e - i);
      i = e;
    } else {
      out += c;
      ++i;
    }
  }
  return out;
}

static bool valid_identifier(const char* s) {
  if (!s || !*s || !(isalpha((unsigned char)*s) || *s == '_')) return false;
  for (const char* p = s; *p; ++p)
    if (!(isalnum((unsigned char)*p) || *p == '_')) return false;
  return true;
}

}  // namespace thb

using namespace thb;

extern "C" {

int thb200_user_kernel_create(const char* name, const char* src, const char* funcs, int nargs,
                              const char* const* arg_names, const int* arg_kinds, thb200_user_kernel** out) {
  if (!out) return fail("user kernel: null output");
  *out = nullptr;
  if (!src || !*src) return fail("Missing parameter src, or was empty");
  const char* kname = (name && *name) ? name : "user_kernel";
  if (!valid_identifier(kname)) return fail("user kernel: `%s` is not a valid kernel name", kname);
  if (nargs < 0 || nargs > 64 || (nargs > 0 && (!arg_names || !arg_kinds))) return fail("user kernel: bad argument list");

  std::unique_ptr<thb200_user_kernel> k(new thb200_user_kernel);
  k->name = kname;
  std::string params, locals;
  for (int i = 0; i < nargs; ++i) {
    if (!valid_identifier(arg_names[i])) return fail("user kernel: `%s` is not a valid argument name", arg_names[i] ? arg_names[i] : "");
    const std::string a = arg_names[i];
    if (i) params += ",\n";
    switch (arg_kinds[i]) {
      case THB200_ARG_INT: params += "    int " + a; break;
      case THB200_ARG_FLOAT: params += "    float " + a; break;
      case THB200_ARG_TENSOR_IN:
      case THB200_ARG_TENSOR_OUT:
      case THB200_ARG_TENSOR_INOUT:
        // the info struct travels by value in the kernel parameters; the body sees a pointer to it
        params += "    const __grid_constant__ THClTensorInfoCl " + a + "_info_v, ";
        params += std::string(arg_kinds[i] == THB200_ARG_TENSOR_IN ? "const " : "") + "float* " + a + "_data";
        locals += "  const THClTensorInfoCl* " + a + "_info = &" + a + "_info_v;\n";
        break;
      default: return fail("user kernel: unknown argument kind %d for `%s`", arg_kinds[i], a.c_str());
    }
    k->kinds.push_back(arg_kinds[i]);
  }
  k->rendered = kOpenClPrelude;
  k->rendered += "\n";
  if (funcs) k->rendered += translate_opencl_words(funcs);
  k->rendered += "\nextern \"C\" __global__ void " + k->name + "(\n" + params + "\n) {\n" + locals +
                 translate_opencl_words(src) + "\n}\n";

  nvrtcProgram prog;
  nvrtcResult r = nvrtcCreateProgram(&prog, k->rendered.c_str(), "thb_user_kernel.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) return fail("NVRTC error in nvrtcCreateProgram: %s", nvrtcGetErrorString(r));
  // functions the user writes without a qualifier are device functions, as in OpenCL C
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--device-as-default-execution-space"};
  r = nvrtcCompileProgram(prog, 3, opts);
  if (r != NVRTC_SUCCESS) {
    size_t logn = 0;
    nvrtcGetProgramLogSize(prog, &logn);
    std::string log(logn, '\0');
    if (logn) nvrtcGetProgramLog(prog, &log[0]);
    nvrtcDestroyProgram(&prog);
    if (log.size() > 1500) log = log.substr(log.size() - 1500);
    return fail("Failed to create kernel %s:\n%s", k->name.c_str(), log.c_str());
  }
  size_t n = 0;
  r = nvrtcGetCUBINSize(prog, &n);
  if (r != NVRTC_SUCCESS || n == 0) { nvrtcDestroyProgram(&prog); return fail("NVRTC error in nvrtcGetCUBINSize: %s", nvrtcGetErrorString(r)); }
  std::vector<char> cubin(n);
  r = nvrtcGetCUBIN(prog, cubin.data());
  nvrtcDestroyProgram(&prog);
  if (r != NVRTC_SUCCESS) return fail("NVRTC error in nvrtcGetCUBIN: %s", nvrtcGetErrorString(r));
  THB_CUDA(cudaGetDevice(&k->device));
  THB_CUDA(cudaLibraryLoadData(&k->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
  cudaError_t e = cudaLibraryGetKernel(&k->kernel, k->lib, k->name.c_str());
  if (e != cudaSuccess) {
    cudaLibraryUnload(k->lib);
    return fail_cuda(e, "cudaLibraryGetKernel(user kernel)");
  }
  *out = k.release();
  return 0;
}

const char* thb200_user_kernel_rendered(const thb200_user_kernel* k) { return k ? k->rendered.c_str() : ""; }

int thb200_user_kernel_run(void* stream, thb200_user_kernel* k, const thb200_user_arg* args, int nargs,
                           int workgroup_size, int64_t num_workgroups) {
  THB_TIMED(stream, "thb200_user_kernel_run");
  if (!k) return fail("user kernel: null kernel");
  if (nargs != (int)k->kinds.size()) return fail("user kernel: %d arguments given, %d declared", nargs, (int)k->kinds.size());
  if (nargs > 0 && !args) return fail("user kernel: null argument array");
  if (workgroup_size < 1 || workgroup_size > 1024) return fail("user kernel: workgroupSize %d out of range (1..1024)", workgroup_size);
  if (num_workgroups < 0 || num_workgroups > 0x7fffffffLL) return fail("user kernel: numWorkgroups out of range");
  if (num_workgroups == 0) return 0;
  int dev = 0;
  THB_CUDA(cudaGetDevice(&dev));
  if (dev != k->device) return fail("user kernel: built for device %d, current device is %d", k->device, dev);

  std::vector<TensorInfoCl> infos(nargs);
  std::vector<void*> ptrs;
  std::vector<const float*> data(nargs);
  std::vector<int> ints(nargs);
  std::vector<float> floats(nargs);
  for (int i = 0; i < nargs; ++i) {
    const thb200_user_arg& a = args[i];
    switch (k->kinds[i]) {
      case THB200_ARG_INT: ints[i] = a.i; ptrs.push_back(&ints[i]); break;
      case THB200_ARG_FLOAT: floats[i] = a.f; ptrs.push_back(&floats[i]); break;
      default: {
        if (a.ndim < 0 || a.ndim > THB200_MAX_DIMS) return fail("user kernel: argument %d has too many dimensions", i);
        if (!a.storage) return fail("user kernel: tensor argument %d has no data", i);
        if (a.offset < 0 || a.offset > 0x7fffffffLL) return fail("user kernel: storage offset of argument %d does not fit an int", i);
        TensorInfoCl& t = infos[i];
        memset(&t, 0, sizeof t);
        for (int d = 0; d < a.ndim; ++d) {
          if (a.size[d] < 0 || a.size[d] > 0xffffffffLL || a.stride[d] < 0 || a.stride[d] > 0xffffffffLL)
            return fail("user kernel: size or stride of argument %d does not fit an unsigned int", i);
          t.sizes[d] = (unsigned int)a.size[d];
          t.strides[d] = (unsigned int)a.stride[d];
        }
        t.offset = (int)a.offset;
        t.dims = a.ndim;
        data[i] = a.storage;
        ptrs.push_back(&t);
        ptrs.push_back(&data[i]);
      }
    }
  }
  THB_CUDA(cudaLaunchKernel((const void*)k->kernel, dim3((unsigned)num_workgroups), dim3((unsigned)workgroup_size),
                            ptrs.empty() ? nullptr : ptrs.data(), 0, (cudaStream_t)stream));
  return 0;
}

void thb200_user_kernel_free(thb200_user_kernel* k) {
  if (!k) return;
  if (k->lib) cudaLibraryUnload(k->lib);
  delete k;
}

}  // extern "C"
