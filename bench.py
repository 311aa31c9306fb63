"""Benchmark of the ClTensor hot path on B200: prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME] [--configs LIST]

Default workload (all N): the sharded large-vector chain — a 2^31-element fp32 vector
(8 GiB, uniform [0,1), seed 4) split evenly over the N GPUs; one step is
    x = x*1.0001 + 0.5 ;  x = sqrt(x) ;  global sum
i.e. two run-time-compiled apply_on_gpu expressions and a reduceAll whose per-GPU partial
is combined across the GPUs and folded in rank order. Algorithmic traffic is 20 bytes per
element (8 + 8 + 4); `value` is that traffic divided by the step time, inputs resident in
HBM. Total work is fixed as N grows ("strong" scaling).

`e2e` times the same step through the C API with the shard starting in pinned host
memory: host->device copy of the shard, the chain, and the 4-byte result read back, every step;
the upload of the next step's shard (second device buffer, copy stream) runs while the kernels
of the current step work.
`check` compares the global sum of that end-to-end step with a double-precision sum
computed on the host from the same pinned shards (1e-5 relative); the run exits non-zero
when it fails. The vector is drawn per fixed block of 2^26 elements, so it is the same
vector at every N.

At N = 1 the line also carries `configs`: benchmark configurations 1-4 (contiguous
map2/sum/div, strided apply, reductions along a dimension with indices and the 100-step
device-resident chain, fp32 GEMM), one entry per operation with its CUDA-event time, its
algorithmic bytes or flops, the fraction of the roofline and a clock record per group
(`--configs ""` leaves them out).

`--impl reference` times the CPU restatement of the reference (oracle/, OpenMP, all host
cores) on the whole 2^31-element vector; the reference itself (OpenCL + Torch7) cannot run
on this box. `--workload c1|c2|c3|c4|n1|n3` (and the smaller `c2small|c3small|c4small|
c4batched|n3small` used for profiler captures) prints one group alone.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from bench_configs import ClockSampler, measured_peaks, run_groups  # noqa: E402

N_TOTAL = 1 << 31
BLOCK = 1 << 26             # the vector is drawn block by block: block b comes from PCG64(4).jumped(b)
BYTES_PER_ELT = 20          # apply 8 + apply 8 + reduce 4
EXPR1 = "x = x*1.0001 + 0.5"
EXPR2 = "x = sqrt(x)"

# dram__bytes_read.sum + dram__bytes_write.sum of one profiler capture of thb_apply_contig on 2^28
# elements (1.073748 GB read + 1.015486 GB written), per element. Taken from that capture, not
# measured in the run; this kernel's DRAM traffic grows in proportion to the element count.
NCU_DRAM_BYTES_PER_ELT_APPLY = (1.073748e9 + 1.015486e9) / 268435456


def host_threads() -> int:
    """Cores this process may run on (torchrun exports OMP_NUM_THREADS=1, so it is asked of the scheduler)."""
    return len(os.sched_getaffinity(0))


def fill_blocks(dst, begin: int, end: int) -> None:
    """dst[0 : end-begin] = elements [begin, end) of the benchmark vector (uniform [0,1), seed 4)."""
    import numpy as np
    b = begin // BLOCK
    while b * BLOCK < end:
        lo, hi = max(begin, b * BLOCK), min(end, (b + 1) * BLOCK)
        g = np.random.Generator(np.random.PCG64(4).jumped(b))
        if lo == b * BLOCK and hi == (b + 1) * BLOCK:
            dst[lo - begin: hi - begin] = g.random(BLOCK, dtype=np.float32)
        else:
            dst[lo - begin: hi - begin] = g.random(BLOCK, dtype=np.float32)[lo - b * BLOCK: hi - b * BLOCK]
        b += 1


def shared_config(n_total: int, world: int) -> dict:
    """The `config` object both arms print."""
    return {"workload": "c5_sharded_apply_reduceall", "elements": n_total,
            "ops": [EXPR1, EXPR2, "sum (reduceAll), per-GPU partials combined and folded in rank order"],
            "algorithmic_bytes_per_element": BYTES_PER_ELT, "parallelism": f"shard{world}",
            "l2": f"inputs larger than L2 ({4 * n_total // world >> 20} MiB per GPU vs 126 MiB)"}


# ---- CPU leg (oracle port) ---------------------------------------------------------------------

def cpu_vector(n: int):
    """The first n elements of the benchmark vector in host memory whose pages were first touched by
    the OpenMP threads that will work on them."""
    import numpy as np
    from oracle import oracle as O
    L = O.lib()
    L.orc_set_num_threads(host_threads())
    x = np.empty(n, dtype=np.float32)
    L.orc_time_touch(C.c_void_p(x.ctypes.data), n)
    fill_blocks(x, 0, n)
    return x


def cpu_step(x) -> float:
    """One step of the chain on the host cores with the oracle's fp32 loops; returns seconds."""
    from oracle import oracle as O
    L = O.lib()
    ptr, n = C.c_void_p(x.ctypes.data), x.size
    t0 = time.perf_counter()
    L.orc_time_axpb(ptr, n, 1.0001, 0.5)
    L.orc_time_sqrt(ptr, n)
    L.orc_time_sum(ptr, n)
    return time.perf_counter() - t0


def cpu_chain(sample_elems: int, reps: int, threads: int = 0):
    """The chain on a sample of the vector; returns (GB/s from the median step, threads used).
    threads = 0: every core this process may use."""
    from oracle import oracle as O
    L = O.lib()
    x = cpu_vector(sample_elems)
    L.orc_set_num_threads(threads if threads > 0 else host_threads())
    cpu_step(x)
    times = [cpu_step(x) for _ in range(reps)]
    return BYTES_PER_ELT * sample_elems / statistics.median(times) / 1e9, L.orc_num_threads()


def torch_cpu_chain(sample_elems: int, reps: int):
    """A second, independent CPU number: the same chain with PyTorch's CPU kernels on all cores."""
    import numpy as np
    import torch
    threads = host_threads()
    torch.set_num_threads(threads)
    g = np.random.Generator(np.random.PCG64(4))
    x = torch.from_numpy(g.random(sample_elems, dtype=np.float32))
    x.mul_(1.0001).add_(0.5)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        x.mul_(1.0001).add_(0.5)            # two passes: PyTorch has no fused a*x+b in place (28 B/elt moved)
        x.sqrt_()
        float(x.sum())
        times.append(time.perf_counter() - t0)
    return BYTES_PER_ELT * sample_elems / statistics.median(times) / 1e9, threads


def run_reference(args):
    """The reference arm: the CPU restatement on the whole vector, every step one full pass."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    n = args.elements
    x = cpu_vector(n)
    threads = O.lib().orc_num_threads()
    for _ in range(args.warmup):
        cpu_step(x)
    total = sum(cpu_step(x) for _ in range(args.steps))
    value = BYTES_PER_ELT * n * args.steps / total / 1e9
    sample = (f"the whole vector ({n} elements, {4 * n >> 20} MiB) in host memory, one pass per step, "
              f"OpenMP on {threads} threads")
    line = {
        "impl": "reference", "metric": "achieved_hbm_gbs_sharded_apply_reduceall", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": shared_config(n, args.gpus),
        "note": "CPU restatement of the reference path (the reference needs OpenCL + Torch7, absent here)",
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- GPU leg -------------------------------------------------------------------------------------

def host_oracle_block_sums(host, begin: int, n_total: int, threads: int):
    """Double-precision sums of sqrt(float32(float32(h*1.0001f) + 0.5f)) over the fixed 2^26-element blocks
    that this rank's pinned shard `host` (elements [begin, begin+len)) covers: a vector with one entry per
    block of the whole vector, zero for blocks of other ranks. Plain torch CPU arithmetic, no library code."""
    import torch
    torch.set_num_threads(max(1, threads))
    nblocks = (n_total + BLOCK - 1) // BLOCK
    sums = torch.zeros(nblocks, dtype=torch.float64)
    end = begin + host.numel()
    b = begin // BLOCK
    while b * BLOCK < end:
        lo, hi = max(begin, b * BLOCK), min(end, (b + 1) * BLOCK)
        y = host[lo - begin: hi - begin].mul(1.0001).add_(0.5).sqrt_()
        rows = y.numel() // 4096 * 4096
        s = y[:rows].view(-1, 4096).sum(dim=1, dtype=torch.float64)       # one row per thread: fixed order
        sums[b] += math.fsum(s.tolist()) + math.fsum(y[rows:].double().tolist())
        b += 1
    return sums


def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs `python -m torch.distributed.run --nproc-per-node N bench.py --gpus N`")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import cltorch_b200 as cl
    from cltorch_b200.sharded import GlobalSum, shard_bounds

    # binds the library to this GPU and to torch's current stream
    gsum = GlobalSum(exchange=None if args.exchange == "auto" else args.exchange)
    n_total = args.elements
    begin, end = shard_bounds(n_total, world, rank)
    n_local = end - begin

    # shard in pinned host memory (for e2e) and resident on the device (for value)
    host = torch.empty(n_local, dtype=torch.float32, pin_memory=True)
    hview = host.numpy()
    fill_blocks(hview, begin, end)
    x = cl.ClTensor(n_local)
    x.copy(hview)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step(events=None, gs=None, t=None):
        gs = gs or gsum
        t = x if t is None else t
        if events is not None:
            events[0].record()
        t.apply_on_gpu(EXPR1)
        if events is not None:
            events[1].record()
        t.apply_on_gpu(EXPR2)
        if events is not None:
            events[2].record()
        r = gs(t)
        if events is not None:
            events[3].record()
        return r

    # nvidia-smi needs a few hundred ms to deliver its first samples: start it before the
    # warm-up and keep the GPU busy for at least half a second before the timed region
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    w_start = time.time()
    # (a step takes about 7 ms / N; the count is the same on every rank because a step has a collective)
    for k in range(max(args.warmup, 3) + args.clock_warmup * world):
        step()
        if k % 16 == 15:
            torch.cuda.synchronize()
    barrier()
    step_events = [[ev() for _ in range(4)] for _ in range(args.steps)]
    start, stop = ev(), ev()
    barrier()
    start.record()
    for k in range(args.steps):
        result = step(step_events[k])
    stop.record()
    barrier()
    c5_window = [(w_start, time.time())]
    elapsed_ms = start.elapsed_time(stop)
    resident_sum = float(result.s())

    # the same timed region with the other exchange (N > 1): the all-gather through torch.distributed
    alt_ms = None
    if world > 1 and gsum.x is not None:
        other = GlobalSum(exchange="nccl")
        for _ in range(max(args.warmup, 3)):
            step(gs=other)
        a0, a1 = ev(), ev()
        barrier()
        a0.record()
        for _ in range(args.steps):
            step(gs=other)
        a1.record()
        barrier()
        alt_ms = a0.elapsed_time(a1)

    # e2e: host buffer -> device, chain, result back to the host; every step. Two device buffers: the upload of
    # step k+1 (its own stream, THClTensor_copyFloatAsync) runs while the kernels of step k work on the other
    # buffer; a buffer is uploaded into again only after the result of its previous step has reached the host.
    e2e_steps = args.steps
    bufs = (x, cl.ClTensor(n_local))
    compute_stream, copy_stream = torch.cuda.current_stream(), torch.cuda.Stream()
    uploaded = [torch.cuda.Event(), torch.cuda.Event()]

    def upload(k):
        bufs[k % 2].copy_async(hview, copy_stream.cuda_stream)
        uploaded[k % 2].record(copy_stream)

    def run_e2e(count):
        upload(0)
        total = None
        for k in range(count):
            if k + 1 < count:
                upload(k + 1)
            compute_stream.wait_event(uploaded[k % 2])
            total = step(t=bufs[k % 2]).s()          # the device -> host read of the step's result
        return total

    run_e2e(2)
    barrier()
    t0 = time.perf_counter()
    total_e2e = run_e2e(e2e_steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    times = torch.tensor([elapsed_ms, e2e_s * 1e3, alt_ms or 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, alt_ms = times.tolist()
    # every rank's own kernel windows: the step waits for the slowest GPU at the exchange
    mine = torch.tensor([statistics.mean(e[i].elapsed_time(e[i + 1]) for e in step_events) for i in range(3)],
                        dtype=torch.float64, device="cuda")
    per_rank = [torch.zeros_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, mine)
    else:
        per_rank = [mine]
    per_rank = [[round(v, 4) for v in t.tolist()] for t in per_rank]

    # parity of the sharded sum: double-precision host sums of the same pinned shards, block by block
    block_sums = host_oracle_block_sums(host, begin, n_total, host_threads() // world).cuda()
    if world > 1:
        dist.all_reduce(block_sums, op=dist.ReduceOp.SUM)      # every block is non-zero on one rank only: exact
    oracle_sum = math.fsum(block_sums.tolist())
    launches_c5 = args.steps * (2 + gsum.launches_per_call)
    del x, bufs, host, hview
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return

    peaks = measured_peaks()
    ms_per_step = elapsed_ms / args.steps
    value = BYTES_PER_ELT * n_total / (ms_per_step * 1e-3) / 1e9
    k_apply = statistics.mean(e[0].elapsed_time(e[1]) for e in step_events)
    k_apply2 = statistics.mean(e[1].elapsed_time(e[2]) for e in step_events)
    k_sum = statistics.mean(e[2].elapsed_time(e[3]) for e in step_events)
    achieved = 8 * n_local / (k_apply * 1e-3) / 1e9
    rel_err = abs(float(total_e2e) - oracle_sum) / abs(oracle_sum)
    config = shared_config(n_total, world)
    config.update({"elements_per_gpu": n_local, "extra_untimed_warmup_steps": args.clock_warmup * world,
                   "exchange": gsum.exchange})
    if gsum.why_not_p2p:
        config["p2p_exchange_unavailable"] = gsum.why_not_p2p
    if alt_ms:
        config["exchange_alternative"] = {"exchange": "all-gather of one float per rank (torch.distributed), fold in rank order",
                                          "ms_per_step": alt_ms / args.steps,
                                          "value": BYTES_PER_ELT * n_total / (alt_ms / args.steps * 1e-3) / 1e9}
    line = {
        "metric": "achieved_hbm_gbs_sharded_apply_reduceall", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "roofline": {"bound": "hbm", "kernel": "thb_apply_contig<UserOp,1> (x = x*1.0001 + 0.5)",
                     "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "traffic": NCU_DRAM_BYTES_PER_ELT_APPLY * n_local,
                     "traffic_note": "bytes per launch from a committed profiler capture, not measured in this run: "
                                     "dram__bytes_read.sum + dram__bytes_write.sum at 2^28 elements (2.0892 GB), "
                                     "scaled by the elements of a launch",
                     "per_kernel_gbs": {"apply_axpb": achieved, "apply_sqrt": 8 * n_local / (k_apply2 * 1e-3) / 1e9,
                                        "reduce_all_sum": 4 * n_local / (k_sum * 1e-3) / 1e9},
                     "per_kernel_ms": {"apply_axpb": k_apply, "apply_sqrt": k_apply2, "sum_and_exchange": k_sum},
                     "per_rank_kernel_ms": {"columns": ["apply_axpb", "apply_sqrt", "sum_and_exchange"], "ranks": per_rank,
                                            "note": "mean CUDA-event windows on each rank; the third window ends when the "
                                                    "slowest rank's partial has arrived"}},
        "e2e": {"value": BYTES_PER_ELT * n_total / (e2e_ms / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": 4 * n_local, "d2h_bytes_per_step": 4, "steps": e2e_steps,
                "pipeline": "two device buffers; the upload of step k+1 overlaps the kernels of step k; the result of "
                            "every step is read back before its buffer is uploaded into again"},
        "gpu_launches": launches_c5,
        "check": {"global_sum_e2e": float(total_e2e), "oracle_sum": oracle_sum, "rel_err": rel_err,
                  "tolerance": 1e-5, "ok": rel_err <= 1e-5,
                  "what": "sum over all GPUs after ONE step on the uploaded vector, against the double-precision "
                          "sum of sqrt(x*1.0001f + 0.5f) computed on the host from the same pinned shards",
                  "resident_chain_sum": resident_sum,
                  "resident_chain_note": "the device-resident vector is updated in place every step and approaches "
                                         "the fixed point of x -> sqrt(1.0001x + 0.5); this sum does not depend on the input"},
    }
    groups = [g for g in args.configs.split(",") if g] if world == 1 else []
    if groups:
        # the clock sampler keeps running; every group gets the samples of its own timed calls
        res = run_groups(groups, max(args.steps, 20), max(args.warmup, 3), sampler)
        line["configs"] = res
        line["gpu_launches"] += sum(g["timed_calls"] for g in res.values())
    line["clocks"] = sampler.summary(c5_window)
    if world == 1:
        gbs, threads = cpu_chain(1 << 28, 8)
        one, _ = cpu_chain(1 << 25, 3, threads=1)
        tgbs, tthreads = torch_cpu_chain(1 << 27, 5)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"2^28 of the 2^31 elements, median of 8 repetitions, OpenMP on {threads} threads",
                                "one_thread": {"value": one, "unit": "GB/s", "cores": 1,
                                               "sample": "2^25 elements, median of 3 repetitions"},
                                "torch_cpu": {"value": tgbs, "unit": "GB/s", "cores": tthreads,
                                              "sample": "2^27 elements, median of 5 repetitions, counted at the same "
                                                        "20 algorithmic bytes per element"}}
    print(json.dumps(line))
    if not line["check"]["ok"]:
        raise SystemExit(f"sharded sum differs from the host oracle: rel_err {rel_err:.3e}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5")
    ap.add_argument("--configs", default="c1,c2,c3,c4",
                    help="groups of per-operation timings added to the N=1 line (comma separated; empty: none)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "p2p", "nccl"],
                    help="how the per-GPU sums are combined at N > 1 (auto: the library's peer-store exchange where it can be set up)")
    ap.add_argument("--elements", type=int, default=N_TOTAL,
                    help="length of the sharded vector (default 2^31; smaller values are for profiler captures)")
    ap.add_argument("--clock-warmup", type=int, default=64,
                    help="extra untimed steps per GPU before the timed region so that clock samples exist (default 64)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c5":
        run_gpu(args)
    else:
        import bench_configs
        bench_configs.run(args.workload, args.steps, max(args.warmup, 3))


if __name__ == "__main__":
    main()
