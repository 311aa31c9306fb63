"""`save` / `load` in Torch7's binary format: byte-level layout of the envelope (numbers, strings,
booleans, tables: no GPU needed) and of ClTensor / ClStorage payloads as the reference writes them
(src/torch/generic/Tensor.cpp:1290-1346, src/torch/generic/Storage.cpp:255-283), round trips of
views, shared storages, point tensors and tables of tensors.
"""
import struct

import numpy as np
import pytest


def i32(v): return struct.pack("<i", v)
def i64(v): return struct.pack("<q", v)
def f64(v): return struct.pack("<d", v)
def s(text): return i32(len(text)) + text.encode()


def test_envelope_of_lua_values(tmp_path):
    import cltorch_b200 as cl
    p = tmp_path / "v.t7"
    cl.save(p, 3.5)
    assert p.read_bytes() == i32(1) + f64(3.5)
    cl.save(p, "hello")
    assert p.read_bytes() == i32(2) + s("hello")
    cl.save(p, True)
    assert p.read_bytes() == i32(5) + i32(1)
    cl.save(p, None)
    assert p.read_bytes() == i32(0)
    cl.save(p, {"a": 1, "b": False})
    assert p.read_bytes() == (i32(3) + i32(1) + i32(2) + i32(2) + s("a") + i32(1) + f64(1) +
                              i32(2) + s("b") + i32(5) + i32(0))
    assert cl.load(p) == {"a": 1, "b": False}
    inner = [10, 20]
    cl.save(p, {"x": inner, "y": inner})                 # the same table twice: written once, then referenced
    back = cl.load(p)
    assert back["x"] == {1: 10, 2: 20} and back["y"] is back["x"]


@pytest.mark.gpu
def test_tensor_bytes_follow_the_reference(tmp_path):
    import cltorch_b200 as cl
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    t = cl.ClTensor(a)
    p = tmp_path / "t.t7"
    cl.save(p, t)
    want = (i32(4) + i32(1) + s("V 1") + s("torch.ClTensor") +
            i32(2) + i64(2) + i64(3) + i64(3) + i64(1) + i64(1) +          # nDimension, size, stride, offset + 1
            i32(4) + i32(2) + s("V 1") + s("torch.ClStorage") + i64(6) + a.tobytes())
    assert p.read_bytes() == want
    back = cl.load(p)
    assert list(back.size()) == [2, 3] and list(back.stride()) == [3, 1] and back.storageOffset() == 1
    assert np.array_equal(back.float(), a)


@pytest.mark.gpu
def test_round_trips_of_views_shared_storage_and_point_tensors(tmp_path):
    import cltorch_b200 as cl
    a = np.random.Generator(np.random.PCG64(81)).random((6, 8), dtype=np.float32)
    base = cl.ClTensor(a)
    view = base.narrow(1, 2, 3).t()                                          # 8 x 3, strides (1, 8), offset 9
    point = cl.ClTensor().sum(base)
    p = tmp_path / "m.t7"
    cl.save(p, {"base": base, "view": view, "sum": point, "n": 48, "name": "demo", "empty": cl.ClTensor()})
    back = cl.load(p)
    assert np.array_equal(back["base"].float(), a)
    v = back["view"]
    assert list(v.size()) == [8, 3] and list(v.stride()) == [1, 8] and v.storageOffset() == 9
    assert np.array_equal(v.float(), a[1:4].T)
    assert v.storage().cdata_ptr() == back["base"].storage().cdata_ptr()      # one storage in the file, one after loading
    v.fill(7.0)                                                               # so writing through the view shows in the base
    assert np.array_equal(back["base"].float()[1:4], np.full((3, 8), 7.0, np.float32))
    assert back["sum"].dim() == 0 and back["sum"].s() == point.s()
    assert back["n"] == 48 and back["name"] == "demo" and back["empty"].dim() <= 0
    # the whole storage travels, as in the reference, even when the tensor views a part of it
    cl.save(p, view)
    assert len(p.read_bytes()) > 4 * a.size
    storage = base.storage()
    cl.save(p, storage)
    assert np.array_equal(cl.load(p).float(), a.ravel())
