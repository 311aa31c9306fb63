"""Python face of the CPU oracle (oracle/thcl_oracle.c) plus a numpy evaluator for
user expressions.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
leg of bench.py. Nothing under cltorch_b200/ imports it.

Strided views are described as (base_array, offset, sizes, strides) in elements, exactly
the (storage, storageOffset, size, stride) of a THClTensor (0-based offset).
"""
from __future__ import annotations

import ast
import ctypes as C
import re
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libthcl_oracle.so"
_lib = None

MOD = {"copy": 0, "abspow": 1, "nezero": 2, "sqdev": 3}
RED = {"add": 0, "mul": 1, "min": 2, "max": 3, "and": 4, "or": 5}


class _T(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_float)), ("nd", C.c_int), ("size", C.POINTER(C.c_int64)),
                ("stride", C.POINTER(C.c_int64))]


def build() -> Path:
    subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        src = _HERE / "thcl_oracle.c"
        if not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
            build()
        L = C.CDLL(str(_LIB_PATH))
        L.orc_reduce_all.restype = C.c_double
        L.orc_reduce_all.argtypes = [C.c_int, C.c_int, C.POINTER(_T), C.c_double, C.c_float, C.c_double]
        L.orc_apply.argtypes = [C.c_char_p, C.c_int, C.POINTER(_T), C.c_float, C.c_float, C.c_float]
        L.orc_reduce_dim.argtypes = [C.c_int, C.c_int, C.POINTER(_T), C.POINTER(_T), C.c_int, C.c_double, C.c_float]
        L.orc_reduce_dim_index.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
        L.orc_addmm.argtypes = ([C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_int64, C.c_int64,
                                 C.c_float, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_int64]
                                + [C.c_int64] * 3)
        L.orc_collapse.argtypes = [C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int,
                                   C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        L.orc_overlapping.argtypes = [C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        L.orc_index_to_offset.restype = C.c_int64
        L.orc_index_to_offset.argtypes = [C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int64]
        L.orc_var_dim.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
        L.orc_scan.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
        L.orc_renorm_rows.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_float]
        L.orc_dist.restype = C.c_double
        L.orc_dist.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float]
        L.orc_time_sum.restype = C.c_double
        L.orc_time_sum.argtypes = [C.c_void_p, C.c_int64]
        L.orc_time_map2_sqrt.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]
        L.orc_time_axpb.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_float]
        L.orc_time_sqrt.argtypes = [C.c_void_p, C.c_int64]
        L.orc_time_mulc.argtypes = [C.c_void_p, C.c_int64, C.c_float]
        L.orc_time_touch.argtypes = [C.c_void_p, C.c_int64]
        _lib = L
    return _lib


class View:
    """(storage array, 0-based offset, sizes, strides): the layout part of a THClTensor."""

    def __init__(self, base: np.ndarray, offset: int = 0, sizes=None, strides=None):
        assert base.dtype == np.float32 and base.flags.c_contiguous
        self.base = base.reshape(-1)
        self.offset = int(offset)
        self.sizes = list(base.shape if sizes is None else sizes)
        if strides is None:
            strides, z = [], 1
            for s in reversed(self.sizes):
                strides.insert(0, z)
                z *= s
        self.strides = list(strides)

    @classmethod
    def of(cls, arr: np.ndarray) -> "View":
        """A view of a numpy array that shares its memory (any positive strides)."""
        base = arr
        while base.base is not None and isinstance(base.base, np.ndarray):
            base = base.base
        off = (arr.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // 4
        return cls(base.reshape(-1), off, arr.shape, [s // 4 for s in arr.strides])

    def nelement(self) -> int:
        return int(np.prod(self.sizes)) if self.sizes else 0

    def numpy(self) -> np.ndarray:
        """The viewed elements as a numpy (strided) array sharing memory."""
        return np.lib.stride_tricks.as_strided(self.base[self.offset:], shape=self.sizes,
                                               strides=[s * 4 for s in self.strides])

    def _c(self):
        nd = len(self.sizes)
        size = (C.c_int64 * max(nd, 1))(*self.sizes)
        stride = (C.c_int64 * max(nd, 1))(*self.strides)
        ptr = C.cast(self.base.ctypes.data + 4 * self.offset, C.POINTER(C.c_float))
        return _T(ptr, nd, size, stride), (size, stride)


def collapse(sizes, strides, reduce_dim: int = -1):
    nd = len(sizes)
    s = (C.c_int64 * max(nd, 1))(*sizes)
    st = (C.c_int64 * max(nd, 1))(*strides)
    os_, ost = (C.c_int64 * max(nd, 1))(), (C.c_int64 * max(nd, 1))()
    d = lib().orc_collapse(nd, s, st, reduce_dim, os_, ost)
    return list(os_[:d]), list(ost[:d])


def overlapping(sizes, strides) -> bool:
    nd = len(sizes)
    return bool(lib().orc_overlapping(nd, (C.c_int64 * max(nd, 1))(*sizes), (C.c_int64 * max(nd, 1))(*strides)))


def index_to_offset(sizes, strides, lin: int) -> int:
    nd = len(sizes)
    return lib().orc_index_to_offset(nd, (C.c_int64 * max(nd, 1))(*sizes), (C.c_int64 * max(nd, 1))(*strides), lin)


def apply(op: str, views, val1: float = 0.0, val2: float = 0.0, point: float = 0.0) -> None:
    """In-place on views[0], as THClTensor_pointwiseApply with the built-in operator `op`."""
    arr = (_T * len(views))()
    keep = []
    for k, v in enumerate(views):
        arr[k], ka = v._c()
        keep.append(ka)
    rc = lib().orc_apply(op.encode(), len(views), arr, val1, val2, point)
    if rc:
        raise ValueError(f"oracle apply {op}: error {rc}")


def reduce_all(view: View, mod: str = "copy", red: str = "add", init: float = 0.0, mod_param: float = 0.0,
               mod_point: float = 0.0) -> float:
    t, keep = view._c()
    return lib().orc_reduce_all(MOD[mod], RED[red], C.byref(t), init, mod_param, mod_point)


def reduce_dim(view: View, dim: int, mod: str = "copy", red: str = "add", init: float = 0.0,
               mod_param: float = 0.0) -> np.ndarray:
    sizes = list(view.sizes)
    sizes[dim] = 1
    out = np.zeros(sizes, dtype=np.float32)
    to, k1 = View(out)._c()
    ti, k2 = view._c()
    rc = lib().orc_reduce_dim(MOD[mod], RED[red], C.byref(to), C.byref(ti), dim, init, mod_param)
    if rc:
        raise ValueError(f"oracle reduce_dim: error {rc}")
    return out


def reduce_dim_index(arr: np.ndarray, dim: int, is_max: bool):
    """(values, 1-based fp32 indices) along `dim` of a contiguous array."""
    a = np.ascontiguousarray(arr, dtype=np.float32)
    outer = int(np.prod(a.shape[:dim])) if dim > 0 else 1
    inner = int(np.prod(a.shape[dim + 1:])) if dim + 1 < a.ndim else 1
    n = a.shape[dim]
    shape = list(a.shape)
    shape[dim] = 1
    values = np.empty(shape, dtype=np.float32)
    indices = np.empty(shape, dtype=np.float32)
    lib().orc_reduce_dim_index(int(is_max), values.ctypes.data, indices.ctypes.data, a.ctypes.data, outer, n, inner)
    return values, indices


def _outer_n_inner(a: np.ndarray, dim: int):
    outer = int(np.prod(a.shape[:dim])) if dim > 0 else 1
    inner = int(np.prod(a.shape[dim + 1:])) if dim + 1 < a.ndim else 1
    return outer, a.shape[dim], inner


def var_dim(arr: np.ndarray, dim: int, flag: bool = False, apply_sqrt: bool = False) -> np.ndarray:
    """var / std along `dim` (size 1 kept), reference src/lib/THClTensorMath2.cl:5-108."""
    a = np.ascontiguousarray(arr, dtype=np.float32)
    outer, n, inner = _outer_n_inner(a, dim)
    shape = list(a.shape)
    shape[dim] = 1
    out = np.empty(shape, dtype=np.float32)
    lib().orc_var_dim(int(flag), int(apply_sqrt), out.ctypes.data, a.ctypes.data, outer, n, inner)
    return out


def scan(arr: np.ndarray, dim: int, is_mul: bool = False) -> np.ndarray:
    """cumsum / cumprod along `dim`, reference src/lib/THClTensorMathScan.cl:27-50."""
    a = np.ascontiguousarray(arr, dtype=np.float32)
    outer, n, inner = _outer_n_inner(a, dim)
    out = np.empty_like(a)
    lib().orc_scan(int(is_mul), out.ctypes.data, a.ctypes.data, outer, n, inner)
    return out


def renorm(arr: np.ndarray, value: float, dim: int, maxnorm: float) -> np.ndarray:
    """renorm as src/lib/THClTensorMath2.cpp:414-446: transpose(dim, 0), contiguous clone, rows rescaled, transposed back."""
    a = np.asarray(arr, dtype=np.float32)
    data = np.array(np.swapaxes(a, dim, 0), dtype=np.float32, order="C", copy=True)
    rows = data.shape[0]
    lib().orc_renorm_rows(data.ctypes.data, rows, data.size // max(rows, 1), value, maxnorm)
    return np.ascontiguousarray(np.swapaxes(data, dim, 0))


def dist(a: np.ndarray, b: np.ndarray, value: float = 2.0) -> float:
    x = np.ascontiguousarray(a, dtype=np.float32).ravel()
    y = np.ascontiguousarray(b, dtype=np.float32).ravel()
    return float(lib().orc_dist(x.ctypes.data, y.ctypes.data, x.size, value))


def addmm(beta: float, t: np.ndarray, alpha: float, m1: np.ndarray, m2: np.ndarray) -> np.ndarray:
    """beta*t + alpha*m1@m2 with fp64 accumulation; 2-D, or 3-D with a leading batch dimension."""
    if m1.ndim == 3:
        return np.stack([addmm(beta, t[b], alpha, m1[b], m2[b]) for b in range(m1.shape[0])])
    M, K = m1.shape
    N = m2.shape[1]
    r = np.empty((M, N), dtype=np.float32)
    t = np.asarray(t, dtype=np.float32)
    s = lambda a: [x // 4 for x in a.strides]
    lib().orc_addmm(r.ctypes.data, N, 1, beta, t.ctypes.data, *s(t), alpha, m1.ctypes.data, *s(m1), m2.ctypes.data,
                    *s(m2), M, N, K)
    return r


# ---- user expressions ------------------------------------------------------------------------
# fp32 arithmetic with one rounding per operation (numpy float32 ops are correctly rounded);
# transcendental functions in float64, rounded once to fp32 — the same policy as the C oracle.

def _f64(fn):
    return lambda *a: fn(*[np.asarray(v, dtype=np.float64) for v in a]).astype(np.float32)


_FUNCS = {
    "sqrt": lambda v: np.sqrt(np.asarray(v, dtype=np.float32)),
    "fabs": lambda v: np.abs(np.asarray(v, dtype=np.float32)), "abs": lambda v: np.abs(np.asarray(v, dtype=np.float32)),
    "floor": lambda v: np.floor(np.asarray(v, dtype=np.float32)), "ceil": lambda v: np.ceil(np.asarray(v, dtype=np.float32)),
    "exp": _f64(np.exp), "log": _f64(np.log), "log1p": _f64(np.log1p), "sin": _f64(np.sin), "cos": _f64(np.cos),
    "tan": _f64(np.tan), "tanh": _f64(np.tanh), "sinh": _f64(np.sinh), "cosh": _f64(np.cosh), "atan": _f64(np.arctan),
    "asin": _f64(np.arcsin), "acos": _f64(np.arccos), "pow": _f64(np.power), "atan2": _f64(np.arctan2),
    "max": lambda a, b: np.fmax(np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)),
    "min": lambda a, b: np.fmin(np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)),
    "fmax": lambda a, b: np.fmax(np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)),
    "fmin": lambda a, b: np.fmin(np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)),
}


def _eval(node, env):
    if isinstance(node, ast.BinOp):
        a, b = _eval(node.left, env), _eval(node.right, env)
        ints = isinstance(a, int) and isinstance(b, int)
        if isinstance(node.op, ast.Add):
            r = a + b
        elif isinstance(node.op, ast.Sub):
            r = a - b
        elif isinstance(node.op, ast.Mult):
            r = a * b
        elif isinstance(node.op, ast.Div):
            r = (a // b) if ints else a / b
        else:
            raise ValueError("unsupported operator")
        return r if ints else np.asarray(r, dtype=np.float32)
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
        v = _eval(node.operand, env)
        return -v
    if isinstance(node, ast.Call):
        return _FUNCS[node.func.id](*[_eval(a, env) for a in node.args])
    if isinstance(node, ast.Name):
        return env[node.id]
    if isinstance(node, ast.Constant):
        if isinstance(node.value, int):
            return node.value  # C integer literal: converts to float only when it meets one
        return np.float32(node.value)
    raise ValueError(f"unsupported syntax: {ast.dump(node)}")


def eval_expr(expr: str, x: np.ndarray, y=None, z=None) -> np.ndarray:
    """Value assigned to x by `x = <expression>` (or the `*out = ...` spelling) in fp32."""
    lhs, rhs = expr.split("=", 1)
    if lhs.strip() not in ("x", "*out", "(*out)"):
        raise ValueError("expression must assign to x")
    rhs = rhs.replace("*out", "x").replace("*in1", "y").replace("*in2", "z")
    rhs = re.sub(r"(?<![\w.])(\d+\.\d*|\.\d+|\d+\.?\d*[eE][+-]?\d+)[fF]?", r"\1", rhs)
    env = {"x": np.asarray(x, dtype=np.float32)}
    if y is not None:
        env["y"] = np.asarray(y, dtype=np.float32)
    if z is not None:
        env["z"] = np.asarray(z, dtype=np.float32)
    out = _eval(ast.parse(rhs.strip(), mode="eval").body, env)
    return np.asarray(out, dtype=np.float32)


def ulp_diff(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between two float32 arrays (NaN == NaN, +0 == -0)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    d = np.abs(ia - ib)
    both_nan = np.isnan(a) & np.isnan(b)
    return np.where(both_nan, 0, d)
