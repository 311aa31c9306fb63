"""cltorch_b200: a B200-native backend for the `torch.ClTensor` hot path of cltorch.

The product is the shared library `cltorch_b200/lib/libthb200.so` (CUDA kernels for
sm_100a behind the C API of include/THCl.h and include/thb200.h); this package is its
ctypes binding plus a `ClTensor` class that mirrors cltorch's Lua methods. Importing the
package does not load the library; the first use does, and fails loudly if it is missing.
"""
from .tensor import (ClError, ClStorage, ClTensor, dumpProfiling, dumpTimings, finish, getDevice, getDeviceCount, getStream,
                     lib, setAddFinish, setDevice, setEnableTiming, setProfiling, setStream, setTrace, state, synchronize)

from .serialization import load, save
from .user_kernel import ClKernel

__all__ = ["ClError", "ClKernel", "ClStorage", "ClTensor", "dumpProfiling", "dumpTimings", "setEnableTiming", "setProfiling", "finish", "getDevice", "getDeviceCount", "getStream", "lib", "load", "save",
           "setAddFinish", "setDevice", "setStream", "setTrace", "state", "synchronize"]
