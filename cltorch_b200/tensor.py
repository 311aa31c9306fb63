"""`ClTensor` / `ClStorage`: the `torch.ClTensor` method surface of cltorch over libthb200.

This is the host-side mirror of cltorch's Lua binding (reference src/TensorMath.lua,
src/Tensor.lua, src/torch/generic/Tensor.cpp): same method names, same overloads and
the same conventions, **including Lua's 1-based dimensions and indices**, so that a test
written against `torch.ClTensor` reads the same here:

    x = ClTensor(a); y = ClTensor(b); z = ClTensor(c)
    x.map2_on_gpu(y, z, "x = sqrt(1000 * x + y * 10 + z * z)")
    s = ClTensor(); s.sum(x)          # point tensor, stays on the GPU
    x.div(s)                          # no host synchronisation anywhere

Every method is one call of the C API in include/THCl.h; nothing is computed in Python.
Host tensors are numpy arrays (`.float()`, `.double()` and `.long()` return them).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import THClState, THClTensor, THClStorage, THLongStorage


class ClError(RuntimeError):
    """An error raised by the C library (the reference raises a Lua error via THError)."""


_L: Optional[C.CDLL] = None
_STATE: Optional[THClState] = None
_HANDLER = None


def lib() -> C.CDLL:
    global _L, _HANDLER
    if _L is None:
        _L = _lib.load()
        # a handler that returns: the failing call comes back and THClLastError() has the message
        _HANDLER = _lib.ERROR_HANDLER(lambda msg, data: None)
        _L.THClSetErrorHandler(_HANDLER, None)
    return _L


def state() -> "C.POINTER(THClState)":
    """The process-wide THClState (cltorch keeps one per Lua state, reference src/init.cpp:234-244)."""
    global _STATE
    if _STATE is None:
        st = THClState()
        lib().THClInit(C.byref(st))
        _STATE = st
        call("THCl_initializeState", C.byref(st))
    return C.byref(_STATE)


def call(name: str, *args):
    L = lib()
    L.THClClearError()
    out = getattr(L, name)(*args)
    err = L.THClLastError()
    if err:
        raise ClError(err.decode())
    return out


# ---- module-level functions of the `cltorch` table (reference src/init.cpp:207-226) ----------

def getDeviceCount() -> int:
    return call("THClState_getNumDevices", state())


def setDevice(device: int) -> None:
    """1-based, as cltorch.setDevice."""
    call("THClState_setDevice", state(), device - 1)


def getDevice() -> int:
    return call("THClState_getDevice", state()) + 1


def synchronize() -> None:
    call("THClSynchronize", state())


finish = synchronize


def setTrace(on: int) -> None:
    state()
    _STATE.trace = int(on)


def setAddFinish(on: int) -> None:
    state()
    _STATE.addFinish = int(on)


def setProfiling(on: int) -> None:
    """cltorch.setProfiling / setEnableTiming (reference src/init.cpp:130-178): device time per library call."""
    lib().thb200_timing_enable(int(on))


setEnableTiming = setProfiling


def dumpProfiling(reset: bool = True) -> dict:
    """cltorch.dumpProfiling / dumpTimings: {entry point: (calls, total milliseconds)} since the last dump."""
    L = lib()
    need = L.thb200_timing_report(None, 0)
    buf = C.create_string_buffer(need + 4096)
    L.thb200_timing_report(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, calls, ms = line.split()
        out[name] = (int(calls), float(ms))
    if reset:
        L.thb200_timing_reset()
    return out


dumpTimings = dumpProfiling


def getStream(device: Optional[int] = None) -> int:
    dev = _STATE.currentDevice if (device is None and _STATE is not None) else ((device or 1) - 1)
    return call("THClState_getStream", state(), dev) or 0


def setStream(stream: int, device: Optional[int] = None) -> None:
    """Makes the library enqueue on a caller-owned CUDA stream (e.g. torch's current stream)."""
    state()
    dev = _STATE.currentDevice if device is None else device - 1
    call("THClState_setStream", state(), dev, C.c_void_p(stream))


def _long_storage(values: Sequence[int]) -> "C.POINTER(THLongStorage)":
    ls = lib().THLongStorage_newWithSize(len(values))
    for k, v in enumerate(values):
        ls.contents.data[k] = int(v)
    return ls


def _host_tensor(arr: np.ndarray, tensor_type, storage_type):
    """A TH<Type>Tensor struct that views a numpy array (kept alive by the returned tuple)."""
    nd = arr.ndim
    item = arr.itemsize
    sizes = (C.c_long * max(nd, 1))(*arr.shape)
    strides = (C.c_long * max(nd, 1))(*[s // item for s in arr.strides])
    st = storage_type()
    st.data = arr.ctypes.data_as(type(st.data))
    st.size = arr.size if nd else 0
    st.refcount = 1
    t = tensor_type()
    t.size, t.stride, t.nDimension = sizes, strides, nd
    t.storage = C.pointer(st)
    t.storageOffset = 0
    t.refcount = 1
    return t, (st, sizes, strides, arr)


class ClStorage:
    """torch.ClStorage (reference src/lib/THClStorage.h)."""

    def __init__(self, arg=None, _ptr=None):
        if _ptr is not None:
            self._p = _ptr
            return
        dev = state()._obj.currentDevice
        if arg is None:
            self._p = call("THClStorage_newv2", state(), dev)
        elif isinstance(arg, (int, np.integer)):
            self._p = call("THClStorage_newWithSize", state(), dev, int(arg))
        else:
            a = np.ascontiguousarray(np.asarray(arg, dtype=np.float32)).ravel()
            self._p = call("THClStorage_newWithSize", state(), dev, a.size)
            if a.size:
                call("THClStorage_rawCopy", state(), self._p, a.ctypes.data_as(C.c_void_p))

    @classmethod
    def from_device_pointer(cls, ptr: int, size: int) -> "ClStorage":
        """Wraps device memory owned by someone else (e.g. a torch CUDA tensor's data_ptr())."""
        dev = state()._obj.currentDevice
        return cls(_ptr=call("THClStorage_newWithDevicePointer", state(), dev, C.c_void_p(ptr), int(size)))

    def __del__(self):
        try:
            if getattr(self, "_p", None):
                lib().THClStorage_free(state(), self._p)
        except Exception:
            pass

    def size(self) -> int:
        return self._p.contents.size

    def fill(self, v: float) -> "ClStorage":
        call("THClStorage_fill", state(), self._p, float(v))
        return self

    def resize(self, n: int) -> "ClStorage":
        call("THClStorage_resize", state(), self._p, int(n))
        return self

    def __getitem__(self, i: int) -> float:
        return call("THClStorage_get", state(), self._p, int(i) - 1)

    def __setitem__(self, i: int, v: float) -> None:
        call("THClStorage_set", state(), self._p, int(i) - 1, float(v))

    def copy(self, src) -> "ClStorage":
        if isinstance(src, ClStorage):
            call("THClStorage_copy", state(), self._p, src._p)
        else:
            a = np.ascontiguousarray(np.asarray(src, dtype=np.float32)).ravel()
            if a.size != self.size():
                raise ClError("bad argument #2: size does not match")
            call("THClStorage_rawCopy", state(), self._p, a.ctypes.data_as(C.c_void_p))
        return self

    def float(self) -> np.ndarray:
        out = np.empty(self.size(), dtype=np.float32)
        hs = _lib.THFloatStorage()
        hs.data = out.ctypes.data_as(_lib.c_float_p)
        hs.size = out.size
        call("THFloatStorage_copyCl", state(), C.byref(hs), self._p)
        return out

    def data_ptr(self) -> int:
        return C.cast(self._p.contents.wrapper, C.c_void_p).value or 0

    def cdata_ptr(self) -> int:
        """Address of the THClStorage struct: two wrappers of one storage compare equal here."""
        return C.cast(self._p, C.c_void_p).value or 0


def _is_tensor(x) -> bool:
    return isinstance(x, ClTensor)


def _is_num(x) -> bool:
    return isinstance(x, (int, float, np.integer, np.floating)) and not isinstance(x, bool)


class ClTensor:
    """torch.ClTensor. Dimensions and indices are 1-based, as in Lua."""

    # ---- construction ---------------------------------------------------------------------
    def __init__(self, *args, _ptr=None):
        if _ptr is not None:
            self._p = _ptr
            return
        dev = state()._obj.currentDevice
        if len(args) == 0:
            self._p = call("THClTensor_newv2", state(), dev)
        elif isinstance(args[0], ClStorage):
            # ClTensor(storage, storageOffset (1-based), sizes, strides)
            storage = args[0]
            offset = int(args[1]) - 1 if len(args) > 1 else 0
            sizes = list(args[2]) if len(args) > 2 else [storage.size()]
            strides = list(args[3]) if len(args) > 3 and args[3] is not None else None
            ls = _long_storage(sizes)
            lst = _long_storage(strides) if strides is not None else None
            try:
                self._p = call("THClTensor_newWithStorage", state(), dev, storage._p, offset, ls, lst)
            finally:
                lib().THLongStorage_free(ls)
                if lst is not None:
                    lib().THLongStorage_free(lst)
        elif all(isinstance(a, (int, np.integer)) for a in args):
            ls = _long_storage(args)
            try:
                self._p = call("THClTensor_newWithSize", state(), dev, ls, None)
            finally:
                lib().THLongStorage_free(ls)
        elif isinstance(args[0], ClTensor):
            self._p = call("THClTensor_newWithTensor", state(), args[0]._p)
        else:
            arr = np.asarray(args[0], dtype=np.float32)
            self._p = call("THClTensor_newv2", state(), dev)
            if arr.size:
                ls = _long_storage(arr.shape)
                try:
                    call("THClTensor_resize", state(), self._p, ls, None)
                finally:
                    lib().THLongStorage_free(ls)
                self.copy(arr)

    def __del__(self):
        try:
            if getattr(self, "_p", None):
                lib().THClTensor_free(state(), self._p)
        except Exception:
            pass

    def _new(self) -> "ClTensor":
        return ClTensor(_ptr=call("THClTensor_newv2", state(), self._p.contents.device))

    # ---- shape ----------------------------------------------------------------------------
    def dim(self) -> int:
        return self._p.contents.nDimension

    nDimension = dim

    def size(self, d: Optional[int] = None):
        t = self._p.contents
        if d is None:
            return tuple(t.size[k] for k in range(max(t.nDimension, 0)))
        return call("THClTensor_size", state(), self._p, d - 1)

    def stride(self, d: Optional[int] = None):
        t = self._p.contents
        if d is None:
            return tuple(t.stride[k] for k in range(max(t.nDimension, 0)))
        return call("THClTensor_stride", state(), self._p, d - 1)

    def storageOffset(self) -> int:
        return self._p.contents.storageOffset + 1

    def storage(self) -> Optional[ClStorage]:
        p = self._p.contents.storage
        if not p:
            return None
        lib().THClStorage_retain(state(), p)
        return ClStorage(_ptr=p)

    def nElement(self) -> int:
        return call("THClTensor_nElement", state(), self._p)

    numel = nElement

    def isContiguous(self) -> bool:
        return bool(call("THClTensor_isContiguous", state(), self._p))

    def isSameSizeAs(self, other: "ClTensor") -> bool:
        return bool(call("THClTensor_isSameSizeAs", state(), self._p, other._p))

    def cdata_ptr(self) -> int:
        """Address of the THClTensor struct."""
        return C.cast(self._p, C.c_void_p).value or 0

    def data_ptr(self) -> int:
        """Device address of the first element."""
        return C.cast(call("THClTensor_data", state(), self._p), C.c_void_p).value or 0

    def resize(self, *sizes) -> "ClTensor":
        if len(sizes) == 1 and not isinstance(sizes[0], (int, np.integer)):
            sizes = tuple(sizes[0])
        ls = _long_storage(sizes)
        try:
            call("THClTensor_resize", state(), self._p, ls, None)
        finally:
            lib().THLongStorage_free(ls)
        return self

    def resizeAs(self, other: "ClTensor") -> "ClTensor":
        call("THClTensor_resizeAs", state(), self._p, other._p)
        return self

    def set(self, other: "ClTensor") -> "ClTensor":
        call("THClTensor_set", state(), self._p, other._p)
        return self

    # views return new tensors that share the storage
    def narrow(self, dim: int, first: int, size: int) -> "ClTensor":
        return ClTensor(_ptr=call("THClTensor_newNarrow", state(), self._p, dim - 1, first - 1, size))

    def select(self, dim: int, index: int) -> "ClTensor":
        return ClTensor(_ptr=call("THClTensor_newSelect", state(), self._p, dim - 1, index - 1))

    def transpose(self, d1: int, d2: int) -> "ClTensor":
        return ClTensor(_ptr=call("THClTensor_newTranspose", state(), self._p, d1 - 1, d2 - 1))

    def t(self) -> "ClTensor":
        if self.dim() != 2:
            raise ClError("Tensor must have 2 dimensions")
        return self.transpose(1, 2)

    def unfold(self, dim: int, size: int, step: int) -> "ClTensor":
        return ClTensor(_ptr=call("THClTensor_newUnfold", state(), self._p, dim - 1, size, step))

    def squeeze(self, dim: Optional[int] = None) -> "ClTensor":
        out = self._new()
        if dim is None:
            call("THClTensor_squeeze", state(), out._p, self._p)
        else:
            call("THClTensor_squeeze1d", state(), out._p, self._p, dim - 1)
        return out

    def expand(self, *sizes) -> "ClTensor":
        """Broadcast view with stride 0 along expanded singleton dimensions (torch.expand)."""
        cur, st = self.size(), self.stride()
        if len(sizes) != len(cur):
            raise ClError("the number of dimensions provided must equal tensor:dim()")
        new_st = []
        for have, s, want in zip(cur, st, sizes):
            if have == want:
                new_st.append(s)
            elif have == 1:
                new_st.append(0)
            else:
                raise ClError("incorrect size: only supporting singleton expansion (size=1)")
        return ClTensor(self.storage(), self.storageOffset(), list(sizes), new_st)

    def clone(self) -> "ClTensor":
        return ClTensor(_ptr=call("THClTensor_newClone", state(), self._p))

    def contiguous(self) -> "ClTensor":
        return ClTensor(_ptr=call("THClTensor_newContiguous", state(), self._p))

    def reshape(self, *sizes) -> "ClTensor":
        out = self._new()
        ls = _long_storage(sizes)
        try:
            call("THClTensor_reshape", state(), out._p, self._p, ls)
        finally:
            lib().THLongStorage_free(ls)
        return out

    # ---- copies ---------------------------------------------------------------------------
    def copy(self, src) -> "ClTensor":
        if _is_tensor(src):
            call("THClTensor_copy", state(), self._p, src._p)
            return self
        arr = np.asarray(src)
        if arr.dtype == np.float64:
            ht, keep = _host_tensor(arr, _lib.THDoubleTensor, _lib.THDoubleStorage)
            call("THClTensor_copyDouble", state(), self._p, C.byref(ht))
        elif arr.dtype == np.int64:
            ht, keep = _host_tensor(arr, _lib.THLongTensor, _lib.THLongStorageH)
            call("THClTensor_copyLong", state(), self._p, C.byref(ht))
        elif arr.dtype == np.int32:
            ht, keep = _host_tensor(arr, _lib.THIntTensor, _lib.THIntStorage)
            call("THClTensor_copyInt", state(), self._p, C.byref(ht))
        elif arr.dtype == np.uint8:
            ht, keep = _host_tensor(arr, _lib.THByteTensor, _lib.THByteStorage)
            call("THClTensor_copyByte", state(), self._p, C.byref(ht))
        else:
            arr = np.asarray(arr, dtype=np.float32)
            ht, keep = _host_tensor(arr, _lib.THFloatTensor, _lib.THFloatStorage)
            call("THClTensor_copyFloat", state(), self._p, C.byref(ht))
        del keep
        return self

    def copy_async(self, src: np.ndarray, stream: int = 0) -> "ClTensor":
        """Upload from a contiguous float32 array in page-locked memory without waiting: the copy is enqueued
        on `stream` (a cudaStream_t as an integer; 0 = the library's current stream); the array must stay alive
        and unchanged until the stream passes it."""
        arr = np.asarray(src)
        if arr.dtype != np.float32 or not arr.flags.c_contiguous:
            raise ClError("copy_async needs a contiguous float32 array")
        call("THClTensor_copyFloatAsync", state(), self._p, C.c_void_p(arr.ctypes.data), int(arr.size), C.c_void_p(stream))
        return self

    def copy_into(self, out: np.ndarray) -> np.ndarray:
        """Device -> host into an existing float32 array (any strides): FloatTensor:copy(clTensor)."""
        ht, keep = _host_tensor(out, _lib.THFloatTensor, _lib.THFloatStorage)
        call("THFloatTensor_copyCl", state(), C.byref(ht), self._p)
        del keep
        return out

    def float(self) -> np.ndarray:
        shape = self.size() if self.dim() > 0 else ()
        if self.dim() == 0:
            return np.float32(self.s())
        out = np.empty(shape, dtype=np.float32)
        if out.size:
            self.copy_into(out)
        return out

    def double(self) -> np.ndarray:
        if self.dim() == 0:
            return np.float64(self.s())
        out = np.empty(self.size(), dtype=np.float64)
        if out.size:
            ht, keep = _host_tensor(out, _lib.THDoubleTensor, _lib.THDoubleStorage)
            call("THDoubleTensor_copyCl", state(), C.byref(ht), self._p)
            del keep
        return out

    def long(self) -> np.ndarray:
        out = np.empty(self.size(), dtype=np.int64)
        if out.size:
            ht, keep = _host_tensor(out, _lib.THLongTensor, _lib.THLongStorageH)
            call("THLongTensor_copyCl", state(), C.byref(ht), self._p)
            del keep
        return out

    # element access, 1-based
    def __getitem__(self, idx):
        idx = idx if isinstance(idx, tuple) else (idx,)
        return call(f"THClTensor_get{len(idx)}d", state(), self._p, *[int(k) - 1 for k in idx])

    def __setitem__(self, idx, value):
        idx = idx if isinstance(idx, tuple) else (idx,)
        call(f"THClTensor_set{len(idx)}d", state(), self._p, *[int(k) - 1 for k in idx], float(value))

    # ---- fills ----------------------------------------------------------------------------
    def fill(self, v) -> "ClTensor":
        if _is_tensor(v):
            call("THClTensor_fill_gpu", state(), self._p, v._p)
        else:
            call("THClTensor_fill", state(), self._p, float(v))
        return self

    def zero(self) -> "ClTensor":
        call("THClTensor_zero", state(), self._p)
        return self

    # ---- user expressions (reference src/TensorMath.lua:591-620) --------------------------
    def apply_on_gpu(self, expr: str) -> "ClTensor":
        call("THClTensor_apply", state(), self._p, expr.encode())
        return self

    def map_on_gpu(self, other: "ClTensor", expr: str) -> "ClTensor":
        call("THClTensor_map", state(), self._p, other._p, expr.encode())
        return self

    def map2_on_gpu(self, a: "ClTensor", b: "ClTensor", expr: str) -> "ClTensor":
        call("THClTensor_map2", state(), self._p, a._p, b._p, expr.encode())
        return self

    apply2_on_gpu = map_on_gpu
    apply3_on_gpu = map2_on_gpu

    # ---- scalar / point-tensor / tensor arithmetic ----------------------------------------
    # Overloads follow the cwrap declarations (reference src/TensorMath.lua:655-736):
    #   add([src,] value) | add([src1,] [value=1,] src2)
    def _scalar_or_tensor(self, args, scalar_fn, tensor_fn, point_fn=None):
        args = list(args)
        if len(args) == 1 and _is_num(args[0]):
            call(scalar_fn, state(), self._p, self._p, float(args[0]))
        elif len(args) == 2 and _is_tensor(args[0]) and _is_num(args[1]):
            call(scalar_fn, state(), self._p, args[0]._p, float(args[1]))
        elif tensor_fn is not None and len(args) >= 1 and _is_tensor(args[-1]):
            src2 = args[-1]
            rest = args[:-1]
            value = 1.0
            src1 = self
            if rest and _is_num(rest[-1]):
                value = float(rest.pop())
            if rest:
                src1 = rest.pop()
            if rest:
                raise ClError("invalid arguments")
            call(tensor_fn, state(), self._p, src1._p, value, src2._p)
        elif point_fn is not None and len(args) >= 1 and _is_tensor(args[-1]):
            src = args[0] if len(args) == 2 else self
            call(point_fn, state(), self._p, src._p, args[-1]._p)
        else:
            raise ClError("invalid arguments")
        return self

    def add(self, *args) -> "ClTensor":
        return self._scalar_or_tensor(args, "THClTensor_add", "THClTensor_cadd")

    def csub(self, *args) -> "ClTensor":
        return self._scalar_or_tensor(args, "THClTensor_sub", "THClTensor_csub")

    sub = csub

    def mul(self, *args) -> "ClTensor":
        return self._scalar_or_tensor(args, "THClTensor_mul", None, "THClTensor_mul_gpu")

    def div(self, *args) -> "ClTensor":
        return self._scalar_or_tensor(args, "THClTensor_div", None, "THClTensor_div_gpu")

    def _binary(self, fn, args):
        if len(args) == 1:
            call(fn, state(), self._p, self._p, args[0]._p)
        else:
            call(fn, state(), self._p, args[0]._p, args[1]._p)
        return self

    def cmul(self, *args) -> "ClTensor":
        return self._binary("THClTensor_cmul", args)

    def cdiv(self, *args) -> "ClTensor":
        return self._binary("THClTensor_cdiv", args)

    def cpow(self, *args) -> "ClTensor":
        return self._binary("THClTensor_cpow", args)

    def cmax(self, *args) -> "ClTensor":
        if _is_num(args[-1]):
            src = args[0] if len(args) == 2 else self
            call("THClTensor_cmaxValue", state(), self._p, src._p, float(args[-1]))
            return self
        return self._binary("THClTensor_cmax", args)

    def cmin(self, *args) -> "ClTensor":
        if _is_num(args[-1]):
            src = args[0] if len(args) == 2 else self
            call("THClTensor_cminValue", state(), self._p, src._p, float(args[-1]))
            return self
        return self._binary("THClTensor_cmin", args)

    def _addc(self, fn, args):
        args = list(args)
        src2 = args.pop()
        src1 = args.pop()
        value = float(args.pop()) if args and _is_num(args[-1]) else 1.0
        t = args.pop() if args else self
        call(fn, state(), self._p, t._p, value, src1._p, src2._p)
        return self

    def addcmul(self, *args) -> "ClTensor":
        return self._addc("THClTensor_addcmul", args)

    def addcdiv(self, *args) -> "ClTensor":
        return self._addc("THClTensor_addcdiv", args)

    def pow(self, *args) -> "ClTensor":
        src = args[0] if len(args) == 2 else self
        call("THClTensor_pow", state(), self._p, src._p, float(args[-1]))
        return self

    def clamp(self, *args) -> "ClTensor":
        src = args[0] if len(args) == 3 else self
        call("THClTensor_clamp", state(), self._p, src._p, float(args[-2]), float(args[-1]))
        return self

    def atan2(self, a: "ClTensor", b: Optional["ClTensor"] = None) -> "ClTensor":
        if b is None:
            a, b = self, a
        call("THClTensor_atan2", state(), self._p, a._p, b._p)
        return self

    def __neg__(self) -> "ClTensor":
        out = self._new()
        call("THClTensor_neg", state(), out._p, self._p)
        return out

    # ---- reductions -----------------------------------------------------------------------
    # sum() -> host float; sum(dim) -> tensor; r:sum(src) with r a tensor -> point tensor
    def _reduce(self, name, args):
        if len(args) == 0:
            return call(f"THClTensor_{name}all", state(), self._p)
        if _is_tensor(args[0]) and len(args) == 1:
            call(f"THClTensor_{name}all_gpu", state(), self._p, args[0]._p)
            return self
        if _is_tensor(args[0]):
            call(f"THClTensor_{name}", state(), self._p, args[0]._p, int(args[1]) - 1)
            return self
        out = self._new()
        call(f"THClTensor_{name}", state(), out._p, self._p, int(args[0]) - 1)
        return out

    def sum(self, *args):
        return self._reduce("sum", args)

    def prod(self, *args):
        return self._reduce("prod", args)

    def mean(self, *args):
        return self._reduce("mean", args)

    def _moment(self, name, args):
        """`x:std()` -> float; `r:std(x)` -> point tensor r; `x:std(dim [, flag])` -> new tensor;
        `r:std(x, dim [, flag])` -> r (reference src/TensorMath.lua:1110-1121)."""
        if len(args) == 0:
            return call(f"THClTensor_{name}all", state(), self._p)
        if _is_tensor(args[0]):
            if len(args) == 1:
                call(f"THClTensor_{name}all_gpu", state(), self._p, args[0]._p)
                return self
            flag = bool(args[2]) if len(args) > 2 else False
            call(f"THClTensor_{name}", state(), self._p, args[0]._p, int(args[1]) - 1, int(flag))
            return self
        flag = bool(args[1]) if len(args) > 1 else False
        out = self._new()
        call(f"THClTensor_{name}", state(), out._p, self._p, int(args[0]) - 1, int(flag))
        return out

    def std(self, *args):
        return self._moment("std", args)

    def var(self, *args):
        return self._moment("var", args)

    def _scan(self, name, args):
        """`x:cumsum(dim)` -> new tensor; `r:cumsum(x, dim)` -> r (reference src/TensorMath.lua:955-962)."""
        if args and _is_tensor(args[0]):
            call(f"THClTensor_{name}", state(), self._p, args[0]._p, int(args[1]) - 1 if len(args) > 1 else 0)
            return self
        out = self._new()
        call(f"THClTensor_{name}", state(), out._p, self._p, int(args[0]) - 1 if args else 0)
        return out

    def cumsum(self, *args):
        return self._scan("cumsum", args)

    def cumprod(self, *args):
        return self._scan("cumprod", args)

    def renorm(self, *args):
        """`x:renorm(p, dim, maxnorm)` -> new tensor; `r:renorm(x, p, dim, maxnorm)` -> r, where r may be x
        (reference src/TensorMath.lua:1136-1142)."""
        if args and _is_tensor(args[0]):
            src, p_, dim, maxnorm = args
            call("THClTensor_renorm", state(), self._p, src._p, float(p_), int(dim) - 1, float(maxnorm))
            return self
        p_, dim, maxnorm = args
        out = self._new()
        call("THClTensor_renorm", state(), out._p, self._p, float(p_), int(dim) - 1, float(maxnorm))
        return out

    def dist(self, other: "ClTensor", value: float = 2.0) -> float:
        return call("THClTensor_dist", state(), self._p, other._p, float(value))

    def dist_gpu(self, a: "ClTensor", b: "ClTensor", value: float = 2.0) -> "ClTensor":
        """self becomes the point tensor holding dist(a, b); no host synchronisation."""
        call("THClTensor_dist_gpu", state(), self._p, a._p, b._p, float(value))
        return self

    def norm(self, value: float = 2.0, dim: Optional[int] = None):
        if dim is None:
            return call("THClTensor_normall", state(), self._p, float(value))
        out = self._new()
        call("THClTensor_norm", state(), out._p, self._p, float(value), dim - 1)
        return out

    def _minmax(self, name, args):
        if len(args) == 0:
            return call(f"THClTensor_{name}all", state(), self._p)
        if _is_tensor(args[0]):
            call(f"THClTensor_{name}all_gpu", state(), self._p, args[0]._p)
            return self
        values, indices = self._new(), self._new()
        call(f"THClTensor_{name}", state(), values._p, indices._p, self._p, int(args[0]) - 1)
        return values, indices

    def max(self, *args):
        return self._minmax("max", args)

    def min(self, *args):
        return self._minmax("min", args)

    def all(self, *args):
        if args:
            call("THClTensor_logicalall_gpu", state(), self._p, args[0]._p)
            return self
        return bool(call("THClTensor_logicalall", state(), self._p))

    def any(self, *args):
        if args:
            call("THClTensor_logicalany_gpu", state(), self._p, args[0]._p)
            return self
        return bool(call("THClTensor_logicalany", state(), self._p))

    def s(self) -> float:
        """Value of a point tensor (`:s()`, reference src/TensorMath.lua:938-941); waits for the GPU."""
        return call("THClTensor_as_float", state(), self._p)

    # ---- BLAS -----------------------------------------------------------------------------
    def _addm(self, fn, args):
        args = list(args)
        m2 = args.pop()
        m1 = args.pop()
        alpha = 1.0
        beta = 1.0
        t = self
        nums = [a for a in args if _is_num(a)]
        tens = [a for a in args if _is_tensor(a)]
        if tens:
            t = tens[0]
        if len(nums) == 1:
            alpha = float(nums[0])
        elif len(nums) == 2:
            beta, alpha = float(nums[0]), float(nums[1])
        call(fn, state(), self._p, beta, t._p, alpha, m1._p, m2._p)
        return self

    def addmm(self, *args) -> "ClTensor":
        """[res] addmm([beta,] [M,] [alpha,] mat1, mat2): res = beta*M + alpha*mat1*mat2."""
        return self._addm("THClTensor_addmm", args)

    def baddbmm(self, *args) -> "ClTensor":
        return self._addm("THClTensor_baddbmm", args)

    def addmv(self, *args) -> "ClTensor":
        """[res] addmv([beta,] [v,] [alpha,] mat, vec): res = beta*v + alpha*mat*vec."""
        return self._addm("THClTensor_addmv", args)

    def addr(self, *args) -> "ClTensor":
        """[res] addr([beta,] [M,] [alpha,] vec1, vec2): res = beta*M + alpha * vec1 (x) vec2."""
        return self._addm("THClTensor_addr", args)

    def mv(self, mat: "ClTensor", vec: "ClTensor") -> "ClTensor":
        self.resize(mat.size(1))
        call("THClTensor_addmv", state(), self._p, 0.0, self._p, 1.0, mat._p, vec._p)
        return self

    def ger(self, v1: "ClTensor", v2: "ClTensor") -> "ClTensor":
        self.resize(v1.size(1), v2.size(1)).zero()
        call("THClTensor_addr", state(), self._p, 1.0, self._p, 1.0, v1._p, v2._p)
        return self

    def dot(self, other: "ClTensor") -> float:
        return call("THClTensor_dot", state(), self._p, other._p)

    def mm(self, m1: "ClTensor", m2: "ClTensor") -> "ClTensor":
        # torch.mm: result zero-initialised, beta = 0 (reference src/TensorMath.lua:827-845)
        self.resize(m1.size(1), m2.size(2))
        call("THClTensor_addmm", state(), self._p, 0.0, self._p, 1.0, m1._p, m2._p)
        return self

    def bmm(self, b1: "ClTensor", b2: "ClTensor") -> "ClTensor":
        self.resize(b1.size(1), b1.size(2), b2.size(3))
        call("THClTensor_baddbmm", state(), self._p, 0.0, self._p, 1.0, b1._p, b2._p)
        return self

    def __repr__(self) -> str:
        return f"ClTensor(size={self.size()}, stride={self.stride()}, offset={self.storageOffset()})"


def _unary(name):
    def method(self, src: Optional[ClTensor] = None) -> ClTensor:
        call(f"THClTensor_{name}", state(), self._p, (src or self)._p)
        return self
    method.__name__ = name
    method.__doc__ = f"self = {name}(src), in place when src is omitted."
    return method


for _n in _lib._UNARY:
    setattr(ClTensor, _n, _unary(_n))


def _compare(name):
    def method(self, a, b=None) -> ClTensor:
        """Out-of-place when called with one argument (returns a new tensor of 0/1), as torch.lt(a, b)."""
        if b is None:
            src, rhs, out = self, a, self._new()
        else:
            src, rhs, out = a, b, self
        if _is_num(rhs):
            call(f"THClTensor_{name}Value", state(), out._p, src._p, float(rhs))
        else:
            call(f"THClTensor_{name}Tensor", state(), out._p, src._p, rhs._p)
        return out
    method.__name__ = name
    return method


for _n in _lib._COMPARE:
    setattr(ClTensor, _n, _compare(_n))
