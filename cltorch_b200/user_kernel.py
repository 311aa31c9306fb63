"""`ClKernel`: user-written kernels, the counterpart of cltorch's `torch.ClKernel`
(reference src/UserKernel.cpp:217-381, README.md:143-215).

    k = ClKernel({"input": {"nElements": "int", "input": "torch.ClTensor"},
                  "output": {"output": "torch.ClTensor"},
                  "src": '''
                     int linearId = get_global_id(0);
                     if(linearId < nElements) {
                       output_data[linearId] = input_data[linearId] + 3.0f;
                     }'''})
    k.run({"nElements": 3, "input": x, "output": y}, {"numWorkgroups": 10, "workgroupSize": 32})

The table keys, the type names, the defaults (64 threads per work-group, one thread per
element of the first output / inout tensor) and the error messages follow the reference.
The body is OpenCL-C-flavoured CUDA: see `thb200_user_kernel_create` in include/thb200.h.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from .tensor import ClError, ClTensor, getStream, state

_KIND = {"int": 0, "float": 1}
_TENSOR_KIND = {"input": 2, "output": 3, "inout": 4}
_DIRECTION_KEYS = {"input": "input", "inputs": "input", "output": "output", "outputs": "output",
                   "inout": "inout", "inouts": "inout"}


class ClKernel:
    def __init__(self, spec: dict):
        if not isinstance(spec, dict):
            raise ClError("First parameter to torch.ClKernel should be a table")
        self.name = "user_kernel"
        self.source = ""
        self.funcs = ""
        self.args = []                      # (name, kind, direction)
        for key, value in spec.items():
            if key in _DIRECTION_KEYS:
                direction = _DIRECTION_KEYS[key]
                for arg, type_name in value.items():
                    if type_name in ("float", "int"):
                        if direction != "input":
                            raise ClError(f"{type_name}s can only be input parameters, not output, or inout")
                        self.args.append((arg, _KIND[type_name], direction))
                    elif type_name in ("torch.ClTensor", "ClTensor"):
                        self.args.append((arg, _TENSOR_KIND[direction], direction))
                    else:
                        raise ClError(f"Unrecognized typename {type_name}")
            elif key == "name":
                self.name = str(value)
            elif key == "src":
                self.source = str(value)
            elif key == "funcs":
                self.funcs = str(value)
            else:
                raise ClError(f"Parameter {key} not recognized")
        if self.source == "":
            raise ClError("Missing parameter src, or was empty")
        L = _lib.load()
        state()                             # a CUDA context on the current device
        names = (C.c_char_p * len(self.args))(*[a[0].encode() for a in self.args])
        kinds = (C.c_int * len(self.args))(*[a[1] for a in self.args])
        handle = C.c_void_p()
        rc = L.thb200_user_kernel_create(self.name.encode(), self.source.encode(), self.funcs.encode(), len(self.args),
                                         names, kinds, C.byref(handle))
        if rc:
            raise ClError(L.thb200_last_error().decode())
        self._h = handle
        self._L = L

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._L.thb200_user_kernel_free(h)

    def getRawKernel(self) -> str:
        return self.source

    def getRenderedKernel(self) -> str:
        return self._L.thb200_user_kernel_rendered(self._h).decode()

    def print(self) -> None:
        print("Original source\n===============\n" + self.source + "\n")
        print("Generated source\n================\n" + self.getRenderedKernel())

    def run(self, params: dict, options: dict | None = None) -> None:
        if not isinstance(params, dict):
            raise ClError("usage  :run(inputParamsTable [,optionsTable]")
        n = len(self.args)
        arr = (_lib.thb200_user_arg * n)()
        keep = []
        num_elements = -1
        for i, (name, kind, direction) in enumerate(self.args):
            if name not in params:
                raise ClError(f"bad argument: field {name} is missing from the parameters table")
            v = params[name]
            if kind == 0:
                arr[i].i = int(v)
            elif kind == 1:
                arr[i].f = float(v)
            else:
                if not isinstance(v, ClTensor):
                    raise ClError(f"bad argument: field {name} is not a torch.ClTensor")
                st = v._p.contents.storage
                base = C.cast(st.contents.wrapper, C.c_void_p).value if st else None
                if not base:
                    raise ClError("Output tensor has no data" if direction != "output" else
                                  "resize not implemented yet.  It should be.  Please remind me to add this, eg raise an issue")
                sizes, strides = list(v.size()), list(v.stride())
                cs = (C.c_int64 * max(len(sizes), 1))(*sizes)
                ct = (C.c_int64 * max(len(strides), 1))(*strides)
                keep += [cs, ct]
                arr[i].storage = C.cast(C.c_void_p(base), _lib.c_float_p)
                arr[i].offset = v.storageOffset() - 1
                arr[i].ndim = len(sizes)
                arr[i].size = cs
                arr[i].stride = ct
                if num_elements == -1 and direction != "input":
                    num_elements = v.nElement()
        if num_elements == -1:
            raise ClError("Must provide at least one output, or inout, ClTensor")
        workgroup_size = 64
        num_workgroups = (num_elements + workgroup_size - 1) // workgroup_size
        if options is not None:
            if not isinstance(options, dict):
                raise ClError("usage  :run(inputParamsTable [,optionsTable]")
            for key, value in options.items():
                if not isinstance(key, str):
                    raise ClError("Options keys should be strings")
                if key == "workgroupSize":
                    if not isinstance(value, (int, float)):
                        raise ClError("workgroupSize should be an integer")
                    workgroup_size = int(value)
                elif key == "numWorkgroups":
                    if not isinstance(value, (int, float)):
                        raise ClError("numWorkgroups should be an integer")
                    num_workgroups = int(value)
                else:
                    raise ClError(f"option {key} not recognized")
        stream = getStream()
        rc = self._L.thb200_user_kernel_run(stream, self._h, arr, n, workgroup_size, num_workgroups)
        if rc:
            raise ClError(self._L.thb200_last_error().decode())
