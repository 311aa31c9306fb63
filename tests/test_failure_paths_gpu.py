"""The give-up path of the bounded device waits, run on purpose in a harmless form.

Every TMA pipeline of the library waits on shared-memory barriers through one routine that gives
up after a time limit, stores a code in the status word of its kernel family and lets the kernel
end. Here a one-warp kernel makes that routine run out on a barrier nothing arrives on (no copy
in flight, a 1 ms limit), and the test checks what a host sees: the kernel returns, the status
call names family and code, the words are cleared, and the next ordinary calls work.
"""
import ctypes as C
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FAMILY_SELFTEST = 6


def test_bounded_wait_runs_out_and_reports_through_the_status_word():
    import cltorch_b200 as cl
    L = cl.lib()
    cl.setDevice(1)
    stream = C.c_void_p(cl.getStream())
    cl.synchronize()
    assert L.thb200_kernel_status(stream) == 0
    t0 = time.perf_counter()
    assert L.thb200_selftest_wait_expiry(stream, 1_000_000, 37) == 0, L.thb200_last_error()
    status = L.thb200_kernel_status(stream)            # synchronises: the kernel has returned by itself
    elapsed = time.perf_counter() - t0
    assert status == 256 * FAMILY_SELFTEST + 37
    assert elapsed < 1.0                                # a 1 ms limit, not the pipelines' 2 s
    assert L.thb200_kernel_status(stream) == 0          # read and cleared
    # the stream and the library are as usable as before
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    A = cl.ClTensor(a)
    assert A.sum() == float(a.sum())
    v, i = A.max(1)
    assert np.array_equal(v.float(), a.max(axis=0, keepdims=True))


def test_status_surfaces_as_an_error_at_the_next_synchronisation():
    import cltorch_b200 as cl
    L = cl.lib()
    cl.setDevice(1)
    stream = C.c_void_p(cl.getStream())
    assert L.thb200_selftest_wait_expiry(stream, 200_000, 5) == 0
    with pytest.raises(cl.ClError, match=r"bounded wait gave up \(self-test, code 5\)"):
        cl.synchronize()
    cl.synchronize()                                     # reported once, then clean again
    assert cl.ClTensor(np.ones(1000, np.float32)).sum() == 1000.0


def test_selftest_rejects_unbounded_limits():
    import cltorch_b200 as cl
    L = cl.lib()
    stream = C.c_void_p(cl.getStream())
    assert L.thb200_selftest_wait_expiry(stream, 0, 1) != 0
    assert L.thb200_selftest_wait_expiry(stream, 5_000_000_000, 1) != 0
    assert L.thb200_selftest_wait_expiry(stream, 1000, 0) != 0
    assert L.thb200_kernel_status(stream) == 0


def test_per_call_device_timing_counts_calls_and_time():
    """cltorch.setProfiling(1) ... cltorch.dumpProfiling(): one bucket per entry point with its call count and
    the device time between the events that bracket its launches."""
    import cltorch_b200 as cl
    cl.setDevice(1)
    a = cl.ClTensor(np.ones((2048, 2048), np.float32))
    b = cl.ClTensor(np.full((2048, 2048), 2.0, np.float32))
    assert cl.dumpProfiling() == {}                       # off: nothing is recorded
    a.add(b)
    assert cl.dumpProfiling() == {}
    cl.setProfiling(1)
    for _ in range(5):
        a.add(b)
    s = cl.ClTensor().sum(a)
    m, i = a.max(1)
    cl.setProfiling(0)
    a.add(b)                                               # not recorded any more
    prof = cl.dumpProfiling()
    assert prof["thb200_apply_op"][0] == 5
    assert prof["thb200_reduce_all"][0] == 1 and prof["thb200_reduce_dim_index"][0] == 1
    # 5 x 48 MiB of traffic cannot take less than 30 us of device time, nor as long as a second
    assert 0.03 < prof["thb200_apply_op"][1] < 1000.0
    assert cl.dumpProfiling() == {}                       # dumped and reset
    assert s.s() == float(2048 * 2048 * 13)                # 1 + six additions of 2 before the sum
