// Instantiates the four apply kernels for every built-in operator of
// apply_ops.def. The file is compiled THB_NPARTS times with -DTHB_PART=k; part k
// instantiates the operators whose code is congruent to k, so the parts build in
// parallel. Part 0 also owns the table and the lookup functions.
#include "thb_internal.h"
#include "../kernels/math_policy.cuh"
#include "../kernels/apply_kernels.cuh"
#include "../kernels/apply_tma_kernels.cuh"

#ifndef THB_NPARTS
#define THB_NPARTS 1
#endif
#ifndef THB_PART
#define THB_PART 0
#endif

namespace thb {

enum BuiltinCode {
#define THB_OP(NAME, NT, ...) OPCODE_##NAME,
#include "../kernels/apply_ops.def"
#undef THB_OP
  OPCODE_COUNT
};

#define THB_OP(NAME, NT, ...)                                                                      \
  struct Op_##NAME {                                                                               \
    static constexpr bool kReadsOut = thb_body_reads_out(#__VA_ARGS__);                            \
    static __device__ __forceinline__ void apply(float* out, const float* in1, const float* in2,   \
                                                 float val1, float val2, const float* pointTensor1, \
                                                 const float* pointTensor2) {                      \
      __VA_ARGS__;                                                                                 \
    }                                                                                              \
  };
#include "../kernels/apply_ops.def"
#undef THB_OP

template <int PART>
static void register_part(ApplyKernels* table) {
#define THB_OP(NAME, NT, ...)                                                        \
  if constexpr (OPCODE_##NAME % THB_NPARTS == PART) {                                \
    ApplyKernels& k = table[OPCODE_##NAME];                                          \
    k.contig = (const void*)&thb_apply_contig<Op_##NAME, NT>;                        \
    k.strided = (const void*)&thb_apply_strided<Op_##NAME, NT>;                      \
    k.tile2d = (const void*)&thb_apply_tile2d<Op_##NAME, NT>;                        \
    k.rows2d = (const void*)&thb_apply_rows2d<Op_##NAME, NT>;                        \
    k.tile2d_v4 = (const void*)&thb_apply_tile2d_v4<Op_##NAME, NT>;                  \
    if constexpr (NT >= 2 || Op_##NAME::kReadsOut)                                   \
      k.tile_tma = (const void*)&thb_apply_tile_tma<Op_##NAME, NT>;                  \
    k.nt = NT;                                                                       \
    k.reads_out = Op_##NAME::kReadsOut;                                              \
    k.name = #NAME;                                                                  \
    k.body = #__VA_ARGS__;                                                           \
  }
#include "../kernels/apply_ops.def"
#undef THB_OP
}

#define THB_CAT2(a, b) a##b
#define THB_CAT(a, b) THB_CAT2(a, b)
void THB_CAT(register_builtin_part_, THB_PART)(ApplyKernels* table) { register_part<THB_PART>(table); }

#if THB_PART == 0
void register_builtin_part_1(ApplyKernels*);
void register_builtin_part_2(ApplyKernels*);
void register_builtin_part_3(ApplyKernels*);
void register_builtin_part_4(ApplyKernels*);
void register_builtin_part_5(ApplyKernels*);
void register_builtin_part_6(ApplyKernels*);
void register_builtin_part_7(ApplyKernels*);

static ApplyKernels* table() {
  static ApplyKernels t[OPCODE_COUNT];
  static bool done = [] {
    register_builtin_part_0(t);
#if THB_NPARTS > 1
    register_builtin_part_1(t);
#endif
#if THB_NPARTS > 2
    register_builtin_part_2(t);
#endif
#if THB_NPARTS > 3
    register_builtin_part_3(t);
#endif
#if THB_NPARTS > 4
    register_builtin_part_4(t);
#endif
#if THB_NPARTS > 5
    register_builtin_part_5(t);
#endif
#if THB_NPARTS > 6
    register_builtin_part_6(t);
#endif
#if THB_NPARTS > 7
    register_builtin_part_7(t);
#endif
    return true;
  }();
  (void)done;
  return t;
}

const ApplyKernels* builtin_op(int code) {
  if (code < 0 || code >= OPCODE_COUNT) return nullptr;
  return &table()[code];
}
int builtin_op_count() { return OPCODE_COUNT; }
#endif

}  // namespace thb
