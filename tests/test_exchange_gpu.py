"""The cross-GPU exchange of per-rank reduction results (thb200_exchange_*) on ONE GPU.

Two ranks of a group live in this process on the same device (their cells are reached through
plain pointers instead of CUDA IPC). All pushes of a step are enqueued before its folds, so no
kernel ever waits for a later launch. The bounded wait is exercised the permitted way: one rank
never pushes, the other's fold gives up after 1 ms, reports through the status word and the
stream stays usable. The path over NVLink between processes is covered by bench.py's check of the
global sum at 2, 4 and 8 GPUs.
"""
import ctypes as C

import numpy as np
import pytest

from cltorch_b200.sharded import tensor_view
from tests.util import rng_uniform

pytestmark = pytest.mark.gpu

RED_ADD, RED_MAX = 0, 3
FAMILY_EXCHANGE = 7


def _group(cl, L, world):
    xs, handles = [], []
    for r in range(world):
        x, h = C.c_void_p(), C.create_string_buffer(128)
        assert L.thb200_exchange_create(r, world, C.byref(x), h) == 0, L.thb200_last_error()
        xs.append(x)
        handles.append(h.raw)
    blob = C.create_string_buffer(b"".join(handles), 128 * world)
    for x in xs:
        assert L.thb200_exchange_connect(x, blob) == 0, L.thb200_last_error()
    return xs


def _scratch(cl, L, n):
    return cl.ClStorage(L.thb200_reduce_all_scratch_bytes(n) // 4 + 16)


def test_two_ranks_on_one_gpu_agree_with_the_plain_reduction_step_after_step():
    import cltorch_b200 as cl
    L = cl.lib()
    cl.setDevice(1)
    stream = C.c_void_p(cl.getStream())
    world = 3
    xs = _group(cl, L, world)
    shards = [rng_uniform(80 + r, (200003 + 1000 * r,), -1, 1) for r in range(world)]
    tensors = [cl.ClTensor(s) for s in shards]
    outs = [cl.ClTensor(1).fill(-1.0) for _ in range(world)]
    sc = _scratch(cl, L, max(s.size for s in shards))
    for step, red in enumerate((RED_ADD, RED_ADD, RED_MAX, RED_ADD)):
        if step == 1:
            for t in tensors:
                t.mul(0.5)
        for r in range(world):                               # every push of the step first ...
            v, keep = tensor_view(tensors[r])
            assert L.thb200_exchange_push(stream, xs[r], red, C.byref(v), C.c_void_p(sc.data_ptr()),
                                          C.c_size_t(sc.size() * 4)) == 0, L.thb200_last_error()
        for r in range(world):                               # ... then the folds: nothing to wait for
            assert L.thb200_exchange_fold(stream, xs[r], red, C.c_void_p(outs[r].data_ptr()), 1_000_000) == 0
        got = [float(o.float()[0]) for o in outs]
        assert got[0] == got[1] == got[2]                    # bit-identical on every rank
        host = [t.float() for t in tensors]
        if red == RED_ADD:
            # the same arithmetic as the single-GPU path: per-shard sums, folded in rank order
            partial = cl.ClTensor(np.array([cl.ClTensor(h).sum() for h in host], np.float32))
            want = partial.sum()
            assert got[0] == want
            ref = sum(float(np.sum(h, dtype=np.float64)) for h in host)
            assert abs(got[0] - ref) <= 1e-5 * max(abs(ref), 1.0)
        else:
            assert got[0] == max(float(h.max()) for h in host)
    assert L.thb200_kernel_status(stream) == 0
    for x in xs:
        assert L.thb200_exchange_destroy(x) == 0


def test_absent_rank_makes_the_bounded_wait_give_up_and_report():
    import cltorch_b200 as cl
    L = cl.lib()
    cl.setDevice(1)
    stream = C.c_void_p(cl.getStream())
    xs = _group(cl, L, 2)
    a = cl.ClTensor(np.ones(5000, np.float32))
    out = cl.ClTensor(1).fill(7.0)
    sc = _scratch(cl, L, 5000)
    v, keep = tensor_view(a)
    # rank 0 pushes, rank 1 never does: rank 0's fold finds one cell missing
    assert L.thb200_exchange_push(stream, xs[0], RED_ADD, C.byref(v), C.c_void_p(sc.data_ptr()), C.c_size_t(sc.size() * 4)) == 0
    assert L.thb200_exchange_fold(stream, xs[0], RED_ADD, C.c_void_p(out.data_ptr()), 1_000_000) == 0
    status = L.thb200_kernel_status(stream)                   # synchronises: the kernel ended by itself
    assert status == 256 * FAMILY_EXCHANGE + 1 + 1            # code = 1 + first missing rank (rank 1)
    assert np.isnan(out.float()[0])
    assert L.thb200_kernel_status(stream) == 0
    assert a.sum() == 5000.0                                  # the stream and the library still work
    # argument checks
    assert L.thb200_exchange_fold(stream, xs[1], RED_ADD, C.c_void_p(out.data_ptr()), 1_000_000) != 0   # no push yet
    assert L.thb200_exchange_fold(stream, xs[0], RED_ADD, C.c_void_p(out.data_ptr()), 0) != 0
    for x in xs:
        L.thb200_exchange_destroy(x)


def _two_gpu_child():
    """One rank of the two-process group below (run through torch.distributed.run)."""
    import os
    import sys
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import cltorch_b200 as cl
    from cltorch_b200.sharded import GlobalSum, shard_bounds
    g = GlobalSum(exchange="p2p", wait_limit_s=5.0)
    n = 3_000_001
    full = np.random.Generator(np.random.PCG64(90)).random(n, dtype=np.float32)
    b, e = shard_bounds(n, 2, rank)
    x = cl.ClTensor(full[b:e])
    got = [float(g(x).s()) for _ in range(3)]               # three steps: both parities of the cells
    ref = float(np.sum(full, dtype=np.float64))
    assert got[0] == got[1] == got[2] and abs(got[0] - ref) <= 1e-5 * ref, (got, ref)
    vals = [None, None]
    dist.all_gather_object(vals, got[0])
    assert vals[0] == vals[1]                                # the same bits on both GPUs
    dist.destroy_process_group()
    print("TWO_GPU_OK")


def test_two_processes_on_two_gpus_over_cuda_ipc():
    """The exchange between processes (CUDA IPC, stores over NVLink). Needs two GPUs; skipped on one."""
    import os
    import subprocess
    import sys
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))   # this file's own imports
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", __file__], capture_output=True, text=True,
                       timeout=300, env=env, cwd=root)
    assert r.returncode == 0 and r.stdout.count("TWO_GPU_OK") == 2, r.stdout[-2000:] + r.stderr[-3000:]


if __name__ == "__main__":
    _two_gpu_child()
