"""`save` / `load` of ClTensors in Torch7's binary file format, as `torch.save(path, clTensor)` /
`torch.load(path)` do with cltorch loaded.

What a ClTensor and a ClStorage put into the file is the reference's own code
(src/torch/generic/Tensor.cpp:1290-1346, src/torch/generic/Storage.cpp:255-283):

    tensor : int nDimension, long size[n], long stride[n], long storageOffset + 1, then the storage
             as an object (or nil)
    storage: long size, float data[size]          (the whole storage, copied to the host)

The envelope around each object is Torch7's `File:writeObject` (torch7/File.lua; Torch7 is a
dependency of the reference and not part of its tree, so this restates the published format):
int type tag (0 nil, 1 number, 2 string, 3 table, 4 torch object, 5 boolean); numbers are
doubles; strings are an int length and the bytes; a table is an int reference index, an int
count and key/value objects; a torch object is an int reference index and, the first time the
index appears, the version string "V 1", the class name and the object's own payload. Objects
referenced twice (two tensors over one storage) are written once. Binary mode, little-endian,
8-byte longs.
"""
from __future__ import annotations

import struct
from typing import Any, BinaryIO

import numpy as np

TYPE_NIL, TYPE_NUMBER, TYPE_STRING, TYPE_TABLE, TYPE_TORCH, TYPE_BOOLEAN = 0, 1, 2, 3, 4, 5


class _Writer:
    def __init__(self, f: BinaryIO):
        self.f = f
        self.index = {}          # identity of an object -> its reference index
        self.keep = []           # objects whose id() is in self.index stay alive

    def i32(self, v): self.f.write(struct.pack("<i", int(v)))
    def i64(self, v): self.f.write(struct.pack("<q", int(v)))
    def f64(self, v): self.f.write(struct.pack("<d", float(v)))

    def string(self, s: str):
        b = s.encode()
        self.i32(len(b))
        self.f.write(b)

    def _ref(self, key, obj) -> bool:
        """Writes the reference index; True if the object still has to be written out."""
        if key in self.index:
            self.i32(self.index[key])
            return False
        self.index[key] = len(self.index) + 1
        self.keep.append(obj)
        self.i32(self.index[key])
        return True

    def obj(self, o: Any):
        from .tensor import ClStorage, ClTensor
        if o is None:
            self.i32(TYPE_NIL)
        elif isinstance(o, bool):
            self.i32(TYPE_BOOLEAN)
            self.i32(1 if o else 0)
        elif isinstance(o, (int, float, np.integer, np.floating)):
            self.i32(TYPE_NUMBER)
            self.f64(o)
        elif isinstance(o, str):
            self.i32(TYPE_STRING)
            self.string(o)
        elif isinstance(o, (dict, list, tuple)):
            self.i32(TYPE_TABLE)
            if self._ref(("table", id(o)), o):
                items = list(o.items()) if isinstance(o, dict) else [(k + 1, v) for k, v in enumerate(o)]
                self.i32(len(items))
                for k, v in items:
                    self.obj(k)
                    self.obj(v)
        elif isinstance(o, ClTensor):
            self.i32(TYPE_TORCH)
            if self._ref(("tensor", o.cdata_ptr()), o):
                self.string("V 1")
                self.string("torch.ClTensor")
                sizes, strides = list(o.size()), list(o.stride())
                self.i32(len(sizes))
                for v in sizes:
                    self.i64(v)
                for v in strides:
                    self.i64(v)
                self.i64(o.storageOffset())              # already 1-based
                self.obj(o.storage())
        elif isinstance(o, ClStorage):
            self.i32(TYPE_TORCH)
            if self._ref(("storage", o.cdata_ptr()), o):
                self.string("V 1")
                self.string("torch.ClStorage")
                data = o.float()
                self.i64(data.size)
                self.f.write(np.ascontiguousarray(data, dtype="<f4").tobytes())
        else:
            raise TypeError(f"cannot serialise {type(o).__name__}")


class _Reader:
    def __init__(self, f: BinaryIO):
        self.f = f
        self.objects = {}

    def _take(self, n):
        b = self.f.read(n)
        if len(b) != n:
            raise EOFError("unexpected end of file")
        return b

    def i32(self): return struct.unpack("<i", self._take(4))[0]
    def i64(self): return struct.unpack("<q", self._take(8))[0]
    def f64(self): return struct.unpack("<d", self._take(8))[0]
    def string(self): return self._take(self.i32()).decode()

    def obj(self):
        from .tensor import ClStorage, ClTensor, call, state
        tag = self.i32()
        if tag == TYPE_NIL:
            return None
        if tag == TYPE_BOOLEAN:
            return self.i32() != 0
        if tag == TYPE_NUMBER:
            v = self.f64()
            return int(v) if v == int(v) and abs(v) < 2 ** 53 else v
        if tag == TYPE_STRING:
            return self.string()
        if tag == TYPE_TABLE:
            idx = self.i32()
            if idx in self.objects:
                return self.objects[idx]
            table = {}
            self.objects[idx] = table
            for _ in range(self.i32()):
                k = self.obj()
                table[k] = self.obj()
            return table
        if tag == TYPE_TORCH:
            idx = self.i32()
            if idx in self.objects:
                return self.objects[idx]
            version = self.string()
            cls = self.string() if version.startswith("V ") else version   # files older than "V 1" have no version
            if cls == "torch.ClStorage":
                n = self.i64()
                data = np.frombuffer(self._take(4 * n), dtype="<f4").astype(np.float32)
                st = ClStorage(data)
                self.objects[idx] = st
                return st
            if cls == "torch.ClTensor":
                nd = self.i32()
                sizes = [self.i64() for _ in range(nd)]
                strides = [self.i64() for _ in range(nd)]
                offset = self.i64()
                storage = self.obj()
                if storage is None:
                    t = ClTensor()
                elif nd > 0:
                    t = ClTensor(storage, offset, sizes, strides)
                else:                                         # a point tensor: no dimensions, one float of storage
                    t = ClTensor()
                    call("THClTensor_setStorage", state(), t._p, storage._p, offset - 1, None, None)
                self.objects[idx] = t
                return t
            raise TypeError(f"cannot read objects of class {cls}")
        raise TypeError(f"unknown type tag {tag}")


def save(path, obj) -> None:
    """`torch.save(path, obj)`: obj may be a ClTensor, a ClStorage, a number, a string, a boolean, None,
    or a dict / list of those (a Lua table)."""
    with open(path, "wb") as f:
        _Writer(f).obj(obj)


def load(path):
    """`torch.load(path)` for files written by `save` (or by Torch7 with cltorch, binary mode)."""
    with open(path, "rb") as f:
        return _Reader(f).obj()
