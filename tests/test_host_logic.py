"""Host-side logic of the library, checked without a GPU: the library loads and exports
every symbol the headers declare; dimension collapsing, the 32-bit-index test, the overlap
test and the kernel plan agree with the oracle and with hand-worked cases; the expression
rewrite; view arithmetic of THClTensor over adopted (never dereferenced) device pointers.
No kernel is launched and no device memory is touched here.
"""
import ctypes as C
import itertools
import json
from pathlib import Path

import numpy as np
import pytest

import __graft_entry__ as entry
from cltorch_b200 import _lib
from oracle import oracle as O

GOLD = json.loads((Path(__file__).parent / "golden" / "reference_known_answers.json").read_text())


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


def arr64(v):
    return (C.c_int64 * max(len(v), 1))(*v)


def test_library_exports_every_declared_symbol(lib):
    declared = entry.declared_symbols()
    assert len(declared) > 200
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    # and the Python prototypes cover the same set
    unbound = sorted(n for n in declared if n not in _lib.PROTOTYPES)
    assert not unbound, unbound


def test_struct_layouts_match_the_ffi_definitions():
    """Field order and offsets of src/FFI.lua:6-33 on LP64."""
    t, s = _lib.THClTensor, _lib.THClStorage
    assert [f[0] for f in t._fields_] == ["size", "stride", "nDimension", "storage", "storageOffset", "refcount", "flag", "device"]
    assert (t.size.offset, t.stride.offset, t.nDimension.offset, t.storage.offset, t.storageOffset.offset,
            t.refcount.offset, t.flag.offset, t.device.offset) == (0, 8, 16, 24, 32, 40, 44, 48)
    assert [f[0] for f in s._fields_] == ["device", "data", "cl", "wrapper", "size", "refcount", "flag", "allocator",
                                          "allocatorContext", "view"]
    assert (s.device.offset, s.data.offset, s.cl.offset, s.wrapper.offset, s.size.offset, s.refcount.offset,
            s.flag.offset, s.allocator.offset) == (0, 8, 16, 24, 32, 40, 44, 48)


def collapse(lib, size, stride, reduce_dim=-1):
    os_, ost = arr64([0] * len(size)), arr64([0] * len(size))
    d = lib.thb200_collapse_dims(len(size), arr64(size), arr64(stride), reduce_dim, os_, ost)
    return list(os_[:d]), list(ost[:d])


@pytest.mark.parametrize("c", GOLD["collapse"], ids=[f"collapse{k}" for k in range(len(GOLD["collapse"]))])
def test_collapse_hand_worked_cases(lib, c):
    assert collapse(lib, c["size"], c["stride"], c["reduce_dim"]) == (c["out_size"], c["out_stride"])


def test_collapse_agrees_with_oracle_on_all_small_layouts(lib):
    """Every permutation / slicing / singleton pattern of up to 4 dims with sizes <= 4."""
    rng = np.random.Generator(np.random.PCG64(50))
    count = 0
    for nd in range(1, 5):
        for sizes in itertools.product([1, 2, 3, 4], repeat=nd):
            for _ in range(3):
                perm = rng.permutation(nd)
                gaps = rng.integers(1, 3, size=nd)
                strides, z = [0] * nd, 1
                for d in perm:                     # a permuted layout with optional holes
                    strides[d] = int(z * gaps[d])
                    z = strides[d] * sizes[d]
                for rd in range(-1, nd):
                    assert collapse(lib, list(sizes), strides, rd) == O.collapse(list(sizes), strides, rd)
                    count += 1
                ov = lib.thb200_overlapping_indices(nd, arr64(sizes), arr64(strides))
                assert bool(ov) == O.overlapping(list(sizes), strides) == False
    assert count > 4000


def test_offsets_of_collapsed_layout_enumerate_the_same_elements():
    """Linear index -> offset through the collapsed dims equals plain row-major enumeration."""
    base = np.arange(4 * 5 * 6, dtype=np.float32).reshape(4, 5, 6)
    for view in (base, base.transpose(2, 0, 1), base[:, 1:4, :], base[:, :, ::2], base[1:3].transpose(1, 0, 2)):
        v = O.View.of(view)
        flat = view.reshape(-1)
        for lin in range(view.size):
            assert base.reshape(-1)[v.offset + O.index_to_offset(v.sizes, v.strides, lin)] == flat[lin]


def test_overlap_detection(lib):
    ov = lambda size, stride: bool(lib.thb200_overlapping_indices(len(size), arr64(size), arr64(stride)))
    assert not ov([4, 3], [3, 1]) and not ov([3, 4], [1, 3]) and not ov([4, 3], [6, 2])
    assert ov([4, 3], [0, 1])            # expanded row
    assert ov([4, 3], [2, 1])            # unfold-like: rows overlap
    assert ov([3], [0])
    assert not ov([1, 1], [0, 0])        # size-1 dims never overlap
    for size, stride in [([4, 3], [0, 1]), ([4, 3], [2, 1]), ([5, 2, 3], [6, 3, 1]), ([5, 2, 3], [3, 3, 1])]:
        assert ov(size, stride) == O.overlapping(size, stride)


def test_32bit_index_limit(lib):
    ok = lambda size, stride: bool(lib.thb200_can_use_32bit_index(len(size), arr64(size), arr64(stride)))
    assert ok([1 << 30], [1]) and ok([1 << 31], [1])
    assert not ok([1 << 32], [1])
    assert ok([1 << 31], [2])                      # last offset 2^32 - 2 is still below UINT_MAX
    assert not ok([1 << 31], [3])
    assert ok([65536, 65535], [65535, 1])
    assert not ok([65536, 65536], [65536, 1])


def plan(lib, layouts):
    ts = (_lib.thb200_tensor * len(layouts))()
    keep = []
    for k, (addr, size, stride) in enumerate(layouts):
        s, st = arr64(size), arr64(stride)
        keep.append((s, st))
        ts[k].data = C.cast(C.c_void_p(addr), _lib.c_float_p)
        ts[k].ndim, ts[k].size, ts[k].stride = len(size), s, st
    return lib.thb200_apply_plan(len(layouts), ts)


def test_kernel_plan(lib):
    A = 0x7F0000000000                              # fake, 16-byte aligned device addresses (never dereferenced)
    n = 8192
    contig = (A, [n, n], [n, 1])
    assert plan(lib, [contig, contig, contig]) == 1                                   # 128-bit contiguous kernel
    assert plan(lib, [(A + 4, [n * n], [1]), (A + 4 + (1 << 30), [n * n], [1])]) == 1     # same phase: still vectorised
    assert plan(lib, [(A, [n * n], [1]), (A + 8, [n * n], [1])]) == 2                  # phases differ: strided kernel
    assert plan(lib, [contig, (A, [n, n], [1, n])]) == 3                               # transpose view: 2-D tile kernel
    assert plan(lib, [(A, [n, n], [1, n]), contig, contig]) == 3                       # transposed destination
    assert plan(lib, [(A, [n, n // 2], [n, 1]), (A, [n, n // 2], [n, 2])]) == 2        # stride-2 slice: 1-D strided
    assert plan(lib, [(A, [4000, n], [n, 1]), (A + 64 * n, [4000, n], [n, 1])]) == 1   # narrowed rows stay one run
    assert plan(lib, [(A, [n, 4000], [n, 1]), (A, [n, 4000], [n, 1])]) == 4            # narrowed columns: 128-bit rows
    assert plan(lib, [(A, [n, 4000], [n, 1]), contig[:1] + ([n, 4000], [4000, 1])]) == 4 # ... mixed with a contiguous one
    assert plan(lib, [(A, [n, 4001], [n, 1]), (A, [n, 4001], [n, 1])]) == 2            # ragged rows: generic strided
    assert plan(lib, [(A + 4, [n, 4000], [n, 1]), (A, [n, 4000], [n, 1])]) == 2        # misaligned rows: generic strided
    assert plan(lib, [(A, [n, 4000], [n, 1]), (A, [n, 4000], [1, n])]) == 3
    assert plan(lib, [(A, [], []), (A, [], [])]) == 0                                  # 0-dim: nothing to do
    assert plan(lib, [(A, [6], [1]), (A, [2, 3], [3, 1])]) == 1                        # equal counts, different shapes
    assert plan(lib, [(A, [6], [1]), (A, [7], [1])]) == -1
    assert b"element size mismatch" in lib.thb200_last_error()
    assert plan(lib, [(A, [1 << 31, 2], [2, 1]), (A, [1 << 31, 2], [2, 1])]) == 1      # 2^32 elements, contiguous: 64-bit counts
    assert plan(lib, [(A, [1 << 31, 2], [4, 1]), (A, [1 << 31, 2], [2, 1])]) == -1     # strided needs 32-bit indices
    assert b"64-bit" in lib.thb200_last_error()


def test_expression_rewrite(lib):
    def rw(expr, nt):
        buf = C.create_string_buffer(1024)
        n = lib.thb200_rewrite_expr(expr.encode(), nt, buf, 1024)
        assert n >= 0
        return buf.value.decode()
    assert rw("x = sqrt(1000*x + y*10 + z*z)", 3) == "(*out) = sqrt(1000*(*out) + (*in1)*10 + (*in2)*(*in2))"
    assert rw("x = exp(x) + max(x, y)", 2) == "(*out) = exp((*out)) + max((*out), (*in1))"       # exp / max survive
    assert rw("x = x + 3.5", 1) == "(*out) = (*out) + 3.5f"
    assert rw("x = x*1.0001 + 0.5", 1) == "(*out) = (*out)*1.0001f + 0.5f"
    assert rw("x = 1e-3 * x + 2.f + .5", 1) == "(*out) = 1e-3f * (*out) + 2.f + .5f"
    assert rw("*out = sqrt(*out + 3) + exp(*out)", 1) == "*out = sqrt(*out + 3) + exp(*out)"     # raw spelling untouched
    assert rw("x = y", 1) == "(*out) = y"                   # y is only an operand name when there is a second tensor
    assert rw("x = xy + y0 + z_", 3) == "(*out) = xy + y0 + z_"
    small = C.create_string_buffer(4)
    assert lib.thb200_rewrite_expr(b"x = x + 1", 1, small, 4) == -1


def test_operator_table(lib):
    for name, arity in [("ADD_3", 3), ("ADD_2", 2), ("FILL_1", 1), ("COPY_2", 2), ("ADDCMUL_3", 3), ("DIVPT_1", 1),
                        ("TANH_2", 2), ("NET_3", 3), ("GEPT_2", 2), ("LTV_2", 2), ("CLAMP_1", 1)]:
        code = lib.thb200_op_code(name.encode())
        assert code >= 0, name
        assert lib.thb200_op_arity(code) == arity
    assert lib.thb200_op_code(b"NOPE_1") == -1


def test_scratch_and_workspace_sizes(lib):
    assert lib.thb200_reduce_all_scratch_bytes(1) == 8
    assert lib.thb200_reduce_all_scratch_bytes(1 << 31) == 592 * 8       # the fixed maximum number of pass-1 blocks
    assert lib.thb200_gemm_workspace_bytes(8192, 8192, 8192, 1) >= 4 * 8192 * 8192 * 4
    assert lib.thb200_reduce_dim_index_scratch_bytes(16384, 16384, 1) == 0


# ---- tensor view arithmetic over an adopted pointer (no device access) --------------------------------

class Host:
    """A THClState that is marked initialised by hand so that nothing asks for a CUDA device."""

    def __init__(self, lib):
        self.lib = lib
        self.state = _lib.THClState()
        lib.THClInit(C.byref(self.state))
        self.state.initialized = 1
        self.state.allocatedDevices = 1
        self.handler = _lib.ERROR_HANDLER(lambda m, d: None)
        lib.THClSetErrorHandler(self.handler, None)
        self.s = C.byref(self.state)

    def tensor(self, size):
        n = int(np.prod(size))
        st = self.lib.THClStorage_newWithDevicePointer(self.s, 0, C.c_void_p(0x7F0000000000), n)
        ls = self.lib.THLongStorage_newWithSize(len(size))
        for k, v in enumerate(size):
            ls.contents.data[k] = v
        t = self.lib.THClTensor_newWithStorage(self.s, 0, st, 0, ls, None)
        self.lib.THLongStorage_free(ls)
        self.lib.THClStorage_free(self.s, st)
        return t

    def meta(self, t):
        c = t.contents
        return ([c.size[k] for k in range(c.nDimension)], [c.stride[k] for k in range(c.nDimension)], c.storageOffset)


def test_view_arithmetic(lib):
    h = Host(lib)
    t = h.tensor([60, 50])
    assert h.meta(t) == ([60, 50], [50, 1], 0)
    assert lib.THClTensor_isContiguous(h.s, t) == 1 and lib.THClTensor_nElement(h.s, t) == 3000
    n = lib.THClTensor_newNarrow(h.s, t, 0, 9, 30)              # Lua narrow(1, 10, 30)
    assert h.meta(n) == ([30, 50], [50, 1], 450) and lib.THClTensor_isContiguous(h.s, n) == 1
    tr = lib.THClTensor_newTranspose(h.s, n, 0, 1)
    assert h.meta(tr) == ([50, 30], [1, 50], 450) and lib.THClTensor_isContiguous(h.s, tr) == 0
    nc = lib.THClTensor_newNarrow(h.s, t, 1, 16, 20)
    assert h.meta(nc) == ([60, 20], [50, 1], 16) and lib.THClTensor_isContiguous(h.s, nc) == 0
    sel = lib.THClTensor_newSelect(h.s, t, 0, 7)
    assert h.meta(sel) == ([50], [1], 350)
    sel2 = lib.THClTensor_newSelect(h.s, t, 1, 7)
    assert h.meta(sel2) == ([60], [50], 7)
    u = lib.THClTensor_newUnfold(h.s, sel, 0, 10, 5)
    assert h.meta(u) == ([9, 10], [5, 1], 350)
    sq = lib.THClTensor_newv2(h.s, 0)
    one = lib.THClTensor_newNarrow(h.s, t, 0, 3, 1)
    lib.THClTensor_squeeze(h.s, sq, one)
    assert h.meta(sq) == ([50], [1], 150)
    # storage is shared and refcounted: 1 (t) + views
    assert t.contents.storage.contents.refcount == 9
    for x in (n, tr, nc, sel, sel2, u, sq, one):
        lib.THClTensor_free(h.s, x)
    assert t.contents.storage.contents.refcount == 1
    # errors come back through the handler, the call returns
    lib.THClClearError()
    bad = lib.THClTensor_newNarrow(h.s, t, 0, 50, 30)
    assert b"out of range" in lib.THClLastError()
    lib.THClClearError()
    lib.THClTensor_free(h.s, t)


def test_empty_and_point_tensor_conventions(lib):
    h = Host(lib)
    e = lib.THClTensor_newv2(h.s, 0)
    assert e.contents.nDimension == -1 and lib.THClTensor_nElement(h.s, e) == 0     # a new tensor has -1 dims
    p = h.tensor([1])
    lib.THClTensor_resize0d(h.s, p)                                                  # point tensor: 0 dims over 1 float
    assert p.contents.nDimension == 0 and lib.THClTensor_nElement(h.s, p) == 0
    assert p.contents.storage.contents.size == 1
    lib.THClTensor_free(h.s, e)
    lib.THClTensor_free(h.s, p)


def test_no_gpu_is_a_loud_error(lib):
    """Without a CUDA device the library refuses to initialise instead of computing on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    st = _lib.THClState()
    lib.THClInit(C.byref(st))
    handler = _lib.ERROR_HANDLER(lambda m, d: None)
    lib.THClSetErrorHandler(handler, None)
    lib.THClClearError()
    lib.THCl_initializeState(C.byref(st))
    assert b"no CUDA device" in lib.THClLastError() and b"no CPU path" in lib.THClLastError()
    assert st.initialized == 0
