"""The multi-GPU path of the sharded vector on CPU ranks: world_size-2 (and 3) gloo process
groups exercise the host logic of cltorch_b200.sharded — shard bounds, the per-rank slot
in the gather buffer, the all-gather and the fixed rank-order fold — with a numpy stand-in
for the device side defined here in the test (the product has no CPU path).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cltorch_b200.sharded import GlobalSum, shard_bounds


def test_shard_bounds_cover_the_vector_exactly():
    for n in (0, 1, 7, 8, 1 << 31, (1 << 31) + 5):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    assert shard_bounds(1 << 31, 8, 3) == (3 << 28, 4 << 28)
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


class NumpyShardOps:
    """Stand-in for the device side: the buffer is a CPU torch tensor, slots are views of it."""

    def new_buffer(self, count):
        buf = torch.zeros(count, dtype=torch.float32)
        return buf, buf

    def slot(self, storage, index):
        return storage[index: index + 1]

    def local_sum_into(self, slot, x):
        slot[0] = float(np.sum(x, dtype=np.float64))

    def fold(self, storage, count, out_slot):
        acc = np.float32(0)
        for r in range(count):                 # rank order, fp32: what thb200_fold_partials does
            acc = np.float32(acc + np.float32(storage[r].item()))
        out_slot[0] = float(acc)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, seed, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = np.random.Generator(np.random.PCG64(seed)).random(n, dtype=np.float32)
        b, e = shard_bounds(n, world, rank)
        gsum = GlobalSum(ops=NumpyShardOps())
        assert gsum.world == world and gsum.rank == rank
        first = float(gsum(full[b:e])[0])
        second = float(gsum(full[b:e] * np.float32(2))[0])      # the buffer is reused call after call
        partials = [float(v) for v in gsum.buf[:world]]
        out[rank] = (first, second, partials, (b, e))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_global_sum_over_gloo_ranks(world):
    n, seed = 1_000_003, 4
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, seed, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    full = np.random.Generator(np.random.PCG64(seed)).random(n, dtype=np.float32)
    want = float(np.sum(full, dtype=np.float64))
    firsts = {out[r][0] for r in range(world)}
    seconds = {out[r][1] for r in range(world)}
    assert len(firsts) == 1 and len(seconds) == 1            # bit-identical on every rank
    assert abs(firsts.pop() - want) <= 1e-5 * want
    assert abs(seconds.pop() - 2 * want) <= 1e-5 * 2 * want
    for r in range(world):                                   # every rank saw every partial, in rank order
        b, e = out[r][3]
        want_r = float(np.sum(full[b:e] * np.float32(2), dtype=np.float64))
        assert abs(out[0][2][r] - want_r) <= 1e-6 * want_r
        assert out[r][2] == out[0][2]


def _worker_with_absent_rank(rank, world, port, out):
    """Rank `world - 1` takes part in the first global sum and then stays away from the second."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    from cltorch_b200.sharded import ExchangeError
    import time
    x = np.full(1000, rank + 1, dtype=np.float32)
    gsum = GlobalSum(ops=NumpyShardOps())
    first = float(gsum(x)[0])
    if rank == world - 1:
        out[rank] = ("absent", first)
        time.sleep(8)                      # alive, but never joins the second exchange
        os._exit(0)                        # no orderly shutdown: its peers have given up on it
    t0 = time.perf_counter()
    try:
        gsum(x)
        out[rank] = ("no error", first)
    except ExchangeError as e:
        out[rank] = ("error", first, time.perf_counter() - t0, str(e))
    os._exit(0)


def test_absent_rank_surfaces_as_a_timeout_error_not_a_hang():
    world = 3
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker_with_absent_rank, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want_first = 1000.0 * (1 + 2 + 3)
    assert out[world - 1] == ("absent", want_first)
    for r in range(world - 1):
        kind, first, waited, msg = out[r]
        assert kind == "error" and first == want_first
        assert waited < 6.0                                   # the 3 s limit of the group, not forever
        assert f"rank {r}" in msg and "exchange" in msg
