"""ctypes binding of libthb200.so: struct layouts and prototypes of include/THCl.h
and include/thb200.h.

The library is the product; there is no Python or CPU fallback. Loading fails
with an ImportError that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "lib" / "libthb200.so"

c_float_p = C.POINTER(C.c_float)
c_long_p = C.POINTER(C.c_long)
c_int64_p = C.POINTER(C.c_int64)


class THLongStorage(C.Structure):
    pass


THLongStorage._fields_ = [
    ("data", c_long_p), ("size", C.c_long), ("refcount", C.c_int), ("flag", C.c_char),
    ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p), ("view", C.POINTER(THLongStorage)),
]


def _host_types(ctype):
    class Storage(C.Structure):
        pass

    Storage._fields_ = [
        ("data", C.POINTER(ctype)), ("size", C.c_long), ("refcount", C.c_int), ("flag", C.c_char),
        ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p), ("view", C.POINTER(Storage)),
    ]

    class Tensor(C.Structure):
        _fields_ = [
            ("size", c_long_p), ("stride", c_long_p), ("nDimension", C.c_int),
            ("storage", C.POINTER(Storage)), ("storageOffset", C.c_long), ("refcount", C.c_int), ("flag", C.c_char),
        ]

    return Storage, Tensor


THFloatStorage, THFloatTensor = _host_types(C.c_float)
THDoubleStorage, THDoubleTensor = _host_types(C.c_double)
THLongStorageH, THLongTensor = _host_types(C.c_long)
THIntStorage, THIntTensor = _host_types(C.c_int)
THByteStorage, THByteTensor = _host_types(C.c_ubyte)


class THClScratchSpace(C.Structure):
    _fields_ = [("wrapper", c_float_p), ("data", c_float_p)]


class THClState(C.Structure):
    _fields_ = [
        ("initialized", C.c_int), ("allowNonGpus", C.c_int), ("allocatedDevices", C.c_int),
        ("currentDevice", C.c_int), ("trace", C.c_int), ("addFinish", C.c_int), ("detailedTimings", C.c_int),
        ("scratchSpaceByDevice", C.c_void_p), ("contextByDevice", C.c_void_p),
    ]


class THClStorage(C.Structure):
    pass


THClStorage._fields_ = [
    ("device", C.c_int), ("data", c_float_p), ("cl", C.c_void_p), ("wrapper", c_float_p), ("size", C.c_long),
    ("refcount", C.c_int), ("flag", C.c_char), ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p),
    ("view", C.POINTER(THClStorage)),
]


class THClTensor(C.Structure):
    _fields_ = [
        ("size", c_long_p), ("stride", c_long_p), ("nDimension", C.c_int), ("storage", C.POINTER(THClStorage)),
        ("storageOffset", C.c_long), ("refcount", C.c_int), ("flag", C.c_char), ("device", C.c_int),
    ]


class thb200_tensor(C.Structure):
    _fields_ = [("data", c_float_p), ("ndim", C.c_int), ("size", c_int64_p), ("stride", c_int64_p)]


class thb200_user_arg(C.Structure):
    _fields_ = [("i", C.c_int), ("f", C.c_float), ("storage", c_float_p), ("offset", C.c_int64), ("ndim", C.c_int),
                ("size", c_int64_p), ("stride", c_int64_p)]


S = C.POINTER(THClState)
ST = C.POINTER(THClStorage)
T = C.POINTER(THClTensor)
LS = C.POINTER(THLongStorage)
f, i, l, v, cp = C.c_float, C.c_int, C.c_long, None, C.c_char_p

ERROR_HANDLER = C.CFUNCTYPE(None, C.c_char_p, C.c_void_p)

_UNARY = ["log", "log1p", "exp", "cos", "acos", "cosh", "sin", "asin", "sinh", "tan", "atan", "tanh", "sqrt",
          "ceil", "floor", "abs", "round", "neg", "cinv", "sigmoid", "sign"]
_COMPARE = ["lt", "gt", "le", "ge", "eq", "ne"]

# name -> (restype, argtypes)
PROTOTYPES = {
    "THClInit": (v, [S]), "THCl_initializeState": (v, [S]), "THClShutdown": (v, [S]),
    "THClSetAllowNonGpus": (v, [S, i]), "THClState_getNumDevices": (i, [S]),
    "THClState_setDevice": (v, [S, i]), "THClState_getDevice": (i, [S]),
    "THClState_getDeviceScratchSpace": (C.POINTER(THClScratchSpace), [S, i, i]),
    "THClState_getDeviceScratchSpaceSize": (C.c_size_t, [S, i]),
    "THClState_getCurrentDeviceScratchSpace": (C.POINTER(THClScratchSpace), [S]),
    "THClState_getCurrentDeviceScratchSpaceSize": (C.c_size_t, [S]),
    "THClSynchronize": (v, [S]), "THClState_getStream": (C.c_void_p, [S, i]),
    "THClState_setStream": (v, [S, i, C.c_void_p]),
    "THClSetErrorHandler": (v, [ERROR_HANDLER, C.c_void_p]), "THClLastError": (cp, []), "THClClearError": (v, []),
    "THLongStorage_newWithSize": (LS, [l]), "THLongStorage_free": (v, [LS]),
    # storage
    "THClStorage_data": (c_float_p, [S, ST]), "THClStorage_size": (l, [S, ST]),
    "THClStorage_set": (v, [S, ST, l, f]), "THClStorage_get": (f, [S, ST, l]),
    "THClStorage_new": (ST, [S]), "THClStorage_newv2": (ST, [S, i]), "THClStorage_newWithSize": (ST, [S, i, l]),
    "THClStorage_newWithSize1": (ST, [S, i, f]), "THClStorage_newWithSize2": (ST, [S, i, f, f]),
    "THClStorage_newWithSize3": (ST, [S, i, f, f, f]), "THClStorage_newWithSize4": (ST, [S, i, f, f, f, f]),
    "THClStorage_newWithData": (ST, [S, i, C.c_void_p, l]),
    "THClStorage_newWithDevicePointer": (ST, [S, i, C.c_void_p, l]),
    "THClStorage_setFlag": (v, [S, ST, C.c_char]), "THClStorage_clearFlag": (v, [S, ST, C.c_char]),
    "THClStorage_retain": (v, [S, ST]), "THClStorage_free": (v, [S, ST]), "THClStorage_resize": (v, [S, ST, l]),
    "THClStorage_fill": (v, [S, ST, f]), "THClStorage_rawCopy": (v, [S, ST, C.c_void_p]),
    "THClStorage_copy": (v, [S, ST, ST]), "THClStorage_copyCl": (v, [S, ST, ST]),
    "THClStorage_copyFloat": (v, [S, ST, C.POINTER(THFloatStorage)]),
    "THFloatStorage_copyCl": (v, [S, C.POINTER(THFloatStorage), ST]),
    # tensor
    "THClTensor_storage": (ST, [S, T]), "THClTensor_storageOffset": (l, [S, T]), "THClTensor_nDimension": (i, [S, T]),
    "THClTensor_size": (l, [S, T, i]), "THClTensor_stride": (l, [S, T, i]),
    "THClTensor_newSizeOf": (LS, [S, T]), "THClTensor_newStrideOf": (LS, [S, T]),
    "THClTensor_data": (c_float_p, [S, T]),
    "THClTensor_wrapper": (c_float_p, [S, T]),
    "THClTensor_setFlag": (v, [S, T, C.c_char]), "THClTensor_clearFlag": (v, [S, T, C.c_char]),
    "THClTensor_new": (T, [S]), "THClTensor_newv2": (T, [S, i]), "THClTensor_newWithTensor": (T, [S, T]),
    "THClTensor_newWithStorage": (T, [S, i, ST, l, LS, LS]),
    "THClTensor_newWithStorage1d": (T, [S, i, ST, l, l, l]),
    "THClTensor_newWithStorage2d": (T, [S, i, ST, l, l, l, l, l]),
    "THClTensor_newWithStorage3d": (T, [S, i, ST, l, l, l, l, l, l, l]),
    "THClTensor_newWithStorage4d": (T, [S, i, ST, l, l, l, l, l, l, l, l, l]),
    "THClTensor_newWithSize": (T, [S, i, LS, LS]), "THClTensor_newWithSize1d": (T, [S, i, l]),
    "THClTensor_newWithSize2d": (T, [S, i, l, l]), "THClTensor_newWithSize3d": (T, [S, i, l, l, l]),
    "THClTensor_newWithSize4d": (T, [S, i, l, l, l, l]),
    "THClTensor_newClone": (T, [S, T]), "THClTensor_newContiguous": (T, [S, T]),
    "THClTensor_newSelect": (T, [S, T, i, l]), "THClTensor_newNarrow": (T, [S, T, i, l, l]),
    "THClTensor_newTranspose": (T, [S, T, i, i]), "THClTensor_newUnfold": (T, [S, T, i, l, l]),
    "THClTensor_resize": (v, [S, T, LS, LS]), "THClTensor_resizeAs": (v, [S, T, T]), "THClTensor_resize0d": (v, [S, T]),
    "THClTensor_resize1d": (v, [S, T, l]), "THClTensor_resize2d": (v, [S, T, l, l]),
    "THClTensor_resize3d": (v, [S, T, l, l, l]), "THClTensor_resize4d": (v, [S, T, l, l, l, l]),
    "THClTensor_resize5d": (v, [S, T, l, l, l, l, l]),
    "THClTensor_set": (v, [S, T, T]), "THClTensor_setStorage": (v, [S, T, ST, l, LS, LS]),
    "THClTensor_setStorage1d": (v, [S, T, ST, l, l, l]), "THClTensor_setStorage2d": (v, [S, T, ST, l, l, l, l, l]),
    "THClTensor_setStorage3d": (v, [S, T, ST, l, l, l, l, l, l, l]),
    "THClTensor_setStorage4d": (v, [S, T, ST, l, l, l, l, l, l, l, l, l]),
    "THClTensor_narrow": (v, [S, T, T, i, l, l]), "THClTensor_select": (v, [S, T, T, i, l]),
    "THClTensor_transpose": (v, [S, T, T, i, i]), "THClTensor_unfold": (v, [S, T, T, i, l, l]),
    "THClTensor_squeeze": (v, [S, T, T]), "THClTensor_squeeze1d": (v, [S, T, T, i]),
    "THClTensor_isContiguous": (i, [S, T]), "THClTensor_isSameSizeAs": (i, [S, T, T]),
    "THClTensor_nElement": (l, [S, T]), "THClTensor_retain": (v, [S, T]), "THClTensor_free": (v, [S, T]),
    "THClTensor_freeCopyTo": (v, [S, T, T]),
    "THClTensor_set1d": (v, [S, T, l, f]), "THClTensor_set2d": (v, [S, T, l, l, f]),
    "THClTensor_set3d": (v, [S, T, l, l, l, f]), "THClTensor_set4d": (v, [S, T, l, l, l, l, f]),
    "THClTensor_get1d": (f, [S, T, l]), "THClTensor_get2d": (f, [S, T, l, l]),
    "THClTensor_get3d": (f, [S, T, l, l, l]), "THClTensor_get4d": (f, [S, T, l, l, l, l]),
    "THClTensor_getDevice": (i, [S, T]), "THClTensor_checkGPU": (i, None),
    # copies
    "THClTensor_copy": (v, [S, T, T]), "THClTensor_copyCl": (v, [S, T, T]),
    "THClTensor_copyIgnoringOverlaps": (v, [S, T, T]),
    "THClTensor_copyFloat": (v, [S, T, C.POINTER(THFloatTensor)]),
    "THClTensor_copyFloatAsync": (v, [S, T, C.c_void_p, l, C.c_void_p]),
    "THFloatTensor_copyCl": (v, [S, C.POINTER(THFloatTensor), T]),
    "THClTensor_copyDouble": (v, [S, T, C.POINTER(THDoubleTensor)]),
    "THDoubleTensor_copyCl": (v, [S, C.POINTER(THDoubleTensor), T]),
    "THClTensor_copyLong": (v, [S, T, C.POINTER(THLongTensor)]),
    "THLongTensor_copyCl": (v, [S, C.POINTER(THLongTensor), T]),
    "THClTensor_copyInt": (v, [S, T, C.POINTER(THIntTensor)]),
    "THIntTensor_copyCl": (v, [S, C.POINTER(THIntTensor), T]),
    "THClTensor_copyByte": (v, [S, T, C.POINTER(THByteTensor)]),
    "THByteTensor_copyCl": (v, [S, C.POINTER(THByteTensor), T]),
    "THClTensor_copyChar": (v, [S, T, C.c_void_p]), "THCharTensor_copyCl": (v, [S, C.c_void_p, T]),
    "THClTensor_copyShort": (v, [S, T, C.c_void_p]), "THShortTensor_copyCl": (v, [S, C.c_void_p, T]),
    # math
    "THClTensor_fill": (v, [S, T, f]), "THClTensor_zero": (v, [S, T]), "THClTensor_zeros": (v, [S, T, LS]),
    "THClTensor_ones": (v, [S, T, LS]), "THClTensor_reshape": (v, [S, T, T, LS]), "THClTensor_numel": (l, [S, T]),
    "THClTensor_add": (v, [S, T, T, f]), "THClTensor_sub": (v, [S, T, T, f]), "THClTensor_mul": (v, [S, T, T, f]),
    "THClTensor_div": (v, [S, T, T, f]),
    "THClTensor_cadd": (v, [S, T, T, f, T]), "THClTensor_csub": (v, [S, T, T, f, T]),
    "THClTensor_cmul": (v, [S, T, T, T]), "THClTensor_cdiv": (v, [S, T, T, T]), "THClTensor_cpow": (v, [S, T, T, T]),
    "THClTensor_addcmul": (v, [S, T, T, f, T, T]), "THClTensor_addcdiv": (v, [S, T, T, f, T, T]),
    "THClTensor_cmin": (v, [S, T, T, T]), "THClTensor_cmax": (v, [S, T, T, T]),
    "THClTensor_cminValue": (v, [S, T, T, f]), "THClTensor_cmaxValue": (v, [S, T, T, f]),
    "THClTensor_pow": (v, [S, T, T, f]), "THClTensor_tpow": (v, [S, T, f, T]),
    "THClTensor_clamp": (v, [S, T, T, f, f]), "THClTensor_atan2": (v, [S, T, T, T]),
    "THClTensor_apply": (v, [S, T, cp]), "THClTensor_map": (v, [S, T, T, cp]), "THClTensor_map2": (v, [S, T, T, T, cp]),
    "THClTensor_add_gpu": (v, [S, T, T, T]), "THClTensor_sub_gpu": (v, [S, T, T, T]),
    "THClTensor_mul_gpu": (v, [S, T, T, T]), "THClTensor_div_gpu": (v, [S, T, T, T]),
    "THClTensor_fill_gpu": (v, [S, T, T]),
    "THClTensor_sumall": (f, [S, T]), "THClTensor_prodall": (f, [S, T]), "THClTensor_minall": (f, [S, T]),
    "THClTensor_maxall": (f, [S, T]), "THClTensor_meanall": (f, [S, T]), "THClTensor_varall": (f, [S, T]),
    "THClTensor_stdall": (f, [S, T]), "THClTensor_normall": (f, [S, T, f]),
    "THClTensor_logicalall": (i, [S, T]), "THClTensor_logicalany": (i, [S, T]), "THClTensor_as_float": (f, [S, T]),
    "THClTensor_sumall_gpu": (v, [S, T, T]), "THClTensor_prodall_gpu": (v, [S, T, T]),
    "THClTensor_minall_gpu": (v, [S, T, T]), "THClTensor_maxall_gpu": (v, [S, T, T]),
    "THClTensor_logicalall_gpu": (v, [S, T, T]), "THClTensor_logicalany_gpu": (v, [S, T, T]),
    "THClTensor_meanall_gpu": (v, [S, T, T]), "THClTensor_varall_gpu": (v, [S, T, T]),
    "THClTensor_stdall_gpu": (v, [S, T, T]),
    "THClTensor_sum": (v, [S, T, T, l]), "THClTensor_prod": (v, [S, T, T, l]), "THClTensor_mean": (v, [S, T, T, l]),
    "THClTensor_norm": (v, [S, T, T, f, l]),
    "THClTensor_var": (v, [S, T, T, l, i]), "THClTensor_std": (v, [S, T, T, l, i]),
    "THClTensor_cumsum": (v, [S, T, T, l]), "THClTensor_cumprod": (v, [S, T, T, l]),
    "THClTensor_renorm": (v, [S, T, T, f, l, f]),
    "THClTensor_dist": (f, [S, T, T, f]), "THClTensor_dist_gpu": (v, [S, T, T, T, f]),
    "THClTensor_max": (v, [S, T, T, T, l]), "THClTensor_min": (v, [S, T, T, T, l]),
    "THClTensor_addmm": (v, [S, T, f, T, f, T, T]), "THClTensor_baddbmm": (v, [S, T, f, T, f, T, T]),
    "THClTensor_addmv": (v, [S, T, f, T, f, T, T]), "THClTensor_addr": (v, [S, T, f, T, f, T, T]),
    "THClTensor_dot": (f, [S, T, T]),
    # thin ABI
    "thb200_last_error": (cp, []),
    "thb200_timing_enable": (v, [i]), "thb200_timing_reset": (v, []),
    "thb200_timing_report": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "thb200_collapse_dims": (i, [i, c_int64_p, c_int64_p, i, c_int64_p, c_int64_p]),
    "thb200_can_use_32bit_index": (i, [i, c_int64_p, c_int64_p]),
    "thb200_overlapping_indices": (i, [i, c_int64_p, c_int64_p]),
    "thb200_apply_plan": (i, [i, C.POINTER(thb200_tensor)]),
    "thb200_op_code": (i, [cp]), "thb200_op_arity": (i, [i]),
    "thb200_apply_op": (i, [C.c_void_p, i, i, C.POINTER(thb200_tensor), f, f, C.c_void_p, C.c_void_p]),
    "thb200_apply_expr": (i, [C.c_void_p, cp, i, C.POINTER(thb200_tensor), f, f, C.c_void_p, C.c_void_p]),
    "thb200_rewrite_expr": (i, [cp, i, C.c_char_p, C.c_size_t]),
    "thb200_reduce_all_scratch_bytes": (C.c_size_t, [C.c_int64]),
    "thb200_reduce_all": (i, [C.c_void_p, i, i, C.POINTER(thb200_tensor), f, f, C.c_void_p, i, f, C.c_void_p,
                              C.c_void_p, C.c_size_t]),
    "thb200_kernel_status": (i, [C.c_void_p]),
    "thb200_selftest_wait_expiry": (i, [C.c_void_p, C.c_uint64, i]),
    "thb200_reduce_dim_scratch_bytes": (C.c_size_t, [C.POINTER(thb200_tensor), i]),
    "thb200_reduce_dim": (i, [C.c_void_p, i, i, C.POINTER(thb200_tensor), C.POINTER(thb200_tensor), i, f, f,
                              C.c_void_p, C.c_size_t]),
    "thb200_reduce_dim_noalloc_capacity": (C.c_size_t, []),
    "thb200_reduce_dim_noalloc": (i, [C.c_void_p, i, i, C.POINTER(thb200_tensor), C.POINTER(thb200_tensor), i, f, f]),
    "thb200_reduce_dim_index": (i, [C.c_void_p, i, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                    C.c_int64, C.c_void_p, C.c_size_t]),
    "thb200_reduce_dim_index_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "thb200_fold_partials": (i, [C.c_void_p, i, C.c_void_p, i, C.c_void_p]),
    "thb200_exchange_create": (i, [i, i, C.POINTER(C.c_void_p), C.c_void_p]),
    "thb200_exchange_connect": (i, [C.c_void_p, C.c_void_p]),
    "thb200_exchange_push": (i, [C.c_void_p, C.c_void_p, i, C.POINTER(thb200_tensor), C.c_void_p, C.c_size_t]),
    "thb200_exchange_fold": (i, [C.c_void_p, C.c_void_p, i, C.c_void_p, C.c_uint64]),
    "thb200_exchange_reduce": (i, [C.c_void_p, C.c_void_p, i, C.POINTER(thb200_tensor), C.c_void_p, C.c_void_p, C.c_size_t,
                                   C.c_uint64]),
    "thb200_exchange_destroy": (i, [C.c_void_p]),
    "thb200_gemm_workspace_bytes": (C.c_size_t, [C.c_int64] * 4),
    "thb200_gemm": (i, [C.c_void_p, C.c_char, C.c_char, C.c_int64, C.c_int64, C.c_int64, f, C.c_void_p, C.c_int64,
                        C.c_void_p, C.c_int64, f, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                        C.c_void_p, C.c_size_t]),
    "thb200_gemm_status": (i, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "thb200_var_dim_scratch_bytes": (C.c_size_t, [C.POINTER(thb200_tensor), i]),
    "thb200_var_dim": (i, [C.c_void_p, C.POINTER(thb200_tensor), C.POINTER(thb200_tensor), i, i, i, C.c_void_p, C.c_size_t]),
    "thb200_var_all_scratch_bytes": (C.c_size_t, [C.c_int64]),
    "thb200_var_all": (i, [C.c_void_p, C.POINTER(thb200_tensor), i, i, C.c_void_p, C.c_void_p, C.c_size_t]),
    "thb200_scan_scratch_bytes": (C.c_size_t, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]),
    "thb200_scan": (i, [C.c_void_p, i, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t,
                        C.c_void_p]),
    "thb200_renorm_rows_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "thb200_renorm_rows": (i, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, f, f, C.c_void_p, C.c_size_t]),
    "thb200_dist_scratch_bytes": (C.c_size_t, [C.c_int64]),
    "thb200_dist": (i, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, f, C.c_void_p, C.c_void_p, C.c_size_t]),
    "thb200_user_kernel_create": (i, [cp, cp, cp, i, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_void_p)]),
    "thb200_user_kernel_rendered": (cp, [C.c_void_p]),
    "thb200_user_kernel_run": (i, [C.c_void_p, C.c_void_p, C.POINTER(thb200_user_arg), i, i, C.c_int64]),
    "thb200_user_kernel_free": (v, [C.c_void_p]),
    "thb200_ger": (i, [C.c_void_p, C.c_int64, C.c_int64, f, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                       C.c_int64, i]),
    "thb200_dot_scratch_bytes": (C.c_size_t, [C.c_int64]),
    "thb200_dot": (i, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_size_t]),
    "thb200_gemv_scratch_bytes": (C.c_size_t, [C.c_char, C.c_int64, C.c_int64]),
    "thb200_gemv": (i, [C.c_void_p, C.c_char, C.c_int64, C.c_int64, f, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, f,
                        C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t]),
}
for _n in _UNARY:
    PROTOTYPES[f"THClTensor_{_n}"] = (v, [S, T, T])
for _n in _COMPARE:
    PROTOTYPES[f"THClTensor_{_n}Value"] = (v, [S, T, T, f])
    PROTOTYPES[f"THClTensor_{_n}Tensor"] = (v, [S, T, T, T])
    PROTOTYPES[f"THClTensor_{_n}PointTensor"] = (v, [S, T, T, T])


def load() -> C.CDLL:
    """Loads the library and sets every prototype; raises ImportError if it is not built."""
    path = Path(os.environ.get("CLTORCH_B200_LIB", LIB_PATH))
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it with `python -m cltorch_b200.build` (needs nvcc for sm_100a). "
            "cltorch_b200 has no CPU or pure-Python fallback.")
    lib = C.CDLL(str(path))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        if args is not None:
            fn.argtypes = args
    return lib
