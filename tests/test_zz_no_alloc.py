"""thb200_reduce_dim_noalloc: the reduction along a dimension for hosts that may not
allocate device memory (its scratch is an array inside the library's device image).

Called through the C ABI and compared bit for bit with thb200_reduce_dim given scratch
from the caller, on two calls in a row that share the built-in array (the second on a
different, smaller shape, so stale partials of the first call would show). The file name
makes pytest collect it last; it also passes when run alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

from cltorch_b200 import _lib
from tests.util import rng_uniform

pytestmark = pytest.mark.gpu

MOD_COPY, RED_ADD, RED_MAX = 0, 0, 3


def _view(tensor, keep):
    """thb200_tensor describing a ClTensor (0-based sizes/strides)."""
    size = (C.c_int64 * max(tensor.dim(), 1))(*tensor.size())
    stride = (C.c_int64 * max(tensor.dim(), 1))(*tensor.stride())
    keep.append((size, stride, tensor))
    t = _lib.thb200_tensor()
    t.data = C.cast(C.c_void_p(tensor.data_ptr()), _lib.c_float_p)
    t.ndim, t.size, t.stride = tensor.dim(), size, stride
    return t


def _reduce_both_ways(cl, L, a, dim, red, init):
    """(result via caller scratch, result via the built-in scratch) for sum/max along `dim` (0-based)."""
    keep = []
    A = cl.ClTensor(a)
    shape = list(a.shape)
    shape[dim] = 1
    out_ref, out_new = cl.ClTensor(*shape).fill(-7.0), cl.ClTensor(*shape).fill(-9.0)
    vin, vref, vnew = _view(A, keep), _view(out_ref, keep), _view(out_new, keep)
    stream = C.c_void_p(cl.getStream())
    need = L.thb200_reduce_dim_scratch_bytes(C.byref(vin), dim)
    scratch = cl.ClStorage(max(need // 4, 1) + 64)
    rc = L.thb200_reduce_dim(stream, MOD_COPY, red, C.byref(vref), C.byref(vin), dim, init, 0.0,
                             C.c_void_p(scratch.data_ptr()), C.c_size_t(scratch.size() * 4))
    assert rc == 0, L.thb200_last_error()
    rc = L.thb200_reduce_dim_noalloc(stream, MOD_COPY, red, C.byref(vnew), C.byref(vin), dim, init, 0.0)
    assert rc == 0, L.thb200_last_error()
    return out_ref.float(), out_new.float(), need


def test_no_alloc_matches_the_allocating_entry_point_twice_in_a_row():
    import cltorch_b200 as cl
    L = cl.lib()
    cl.setDevice(1)
    # first call: a column reduction that is cut into chunks and therefore uses the scratch
    a = rng_uniform(71, (4096, 1000), -1, 1)
    ref, new, need = _reduce_both_ways(cl, L, a, 0, RED_ADD, 0.0)
    assert 0 < need <= L.thb200_reduce_dim_noalloc_capacity()
    assert np.array_equal(ref, new)
    want = a.sum(axis=0, dtype=np.float64, keepdims=True)
    assert np.all(np.abs(new - want) <= 1e-5 * np.maximum(np.abs(want), 1.0))
    # second call right after it, other shape and operator, same built-in array
    b = rng_uniform(72, (3, 700, 130), -1, 1)
    ref, new, need = _reduce_both_ways(cl, L, b, 1, RED_MAX, -np.inf)
    assert np.array_equal(ref, new)
    assert np.array_equal(new, b.max(axis=1, keepdims=True))
    # and once more on the first shape: the answer does not depend on what the array held
    ref2, new2, _ = _reduce_both_ways(cl, L, a, 0, RED_ADD, 0.0)
    assert np.array_equal(new2, ref2) and np.array_equal(new2, _reduce_both_ways(cl, L, a, 0, RED_ADD, 0.0)[1])


def test_no_alloc_call_leaves_free_device_memory_unchanged():
    """The point of the entry point: once its set-up call is over, a call neither takes nor returns device
    memory (the free bytes the driver reports stay the same across it)."""
    import torch
    import cltorch_b200 as cl
    L = cl.lib()
    cl.setDevice(1)
    keep = []
    a = rng_uniform(73, (4096, 1000), -1, 1)
    A = cl.ClTensor(a)
    out = cl.ClTensor(1, 1000)
    vin, vout = _view(A, keep), _view(out, keep)
    stream = C.c_void_p(cl.getStream())
    assert L.thb200_reduce_dim_noalloc(stream, MOD_COPY, RED_ADD, C.byref(vout), C.byref(vin), 0, 0.0, 0.0) == 0   # set-up call
    cl.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(3):
        assert L.thb200_reduce_dim_noalloc(stream, MOD_COPY, RED_ADD, C.byref(vout), C.byref(vin), 0, 0.0, 0.0) == 0
    cl.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before
    want = a.sum(axis=0, dtype=np.float64, keepdims=True)
    assert np.all(np.abs(out.float() - want) <= 1e-5 * np.maximum(np.abs(want), 1.0))


def test_no_alloc_refuses_shapes_beyond_its_scratch():
    import cltorch_b200 as cl
    L = cl.lib()
    cap = L.thb200_reduce_dim_noalloc_capacity()
    assert cap == 4 << 20
    # layout only: nothing is launched because the shape is refused first
    keep = []
    rows, cols = 512, 290000
    size = (C.c_int64 * 2)(rows, cols)
    stride = (C.c_int64 * 2)(cols, 1)
    osize = (C.c_int64 * 2)(1, cols)
    fake = C.cast(C.c_void_p(0x7F0000000000), _lib.c_float_p)
    vin, vout = _lib.thb200_tensor(fake, 2, size, stride), _lib.thb200_tensor(fake, 2, osize, stride)
    need = L.thb200_reduce_dim_scratch_bytes(C.byref(vin), 0)
    assert need > cap
    rc = L.thb200_reduce_dim_noalloc(None, MOD_COPY, RED_ADD, C.byref(vout), C.byref(vin), 0, 0.0, 0.0)
    assert rc != 0
    msg = L.thb200_last_error().decode()
    assert "built-in scratch" in msg and str(need) in msg
