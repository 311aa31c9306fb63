"""Benchmark of the ClTensor hot path on B200: prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload (all N): the sharded large-vector chain — a 2^31-element fp32 vector
(8 GiB, uniform [0,1), seed 4) split evenly over the N GPUs; one step is
    x = x*1.0001 + 0.5 ;  x = sqrt(x) ;  global sum
i.e. two run-time-compiled apply_on_gpu expressions and a reduceAll whose per-GPU partial
is combined by an all-gather over NCCL and a fixed-order fold. Algorithmic traffic is
20 bytes per element (8 + 8 + 4); `value` is that traffic divided by the step time,
inputs resident in HBM. Total work is fixed as N grows ("strong" scaling).

`e2e` times the same step through the C API with the shard starting in pinned host
memory: host->device copy of the shard, the chain, and the 4-byte result read back.

`--impl reference` times the CPU restatement of the reference (oracle/, OpenMP, all host
cores) on a bounded sample of the same workload; the reference itself (OpenCL + Torch7)
cannot run on this box. Other workloads (`--workload c1|c2|c3|c4|n3`, and the smaller
`c2small|c3small|c4small|c4batched|n3small` used for profiler captures) report the remaining
benchmark configurations at N=1; they are not the driver's default line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_TOTAL = 1 << 31
BYTES_PER_ELT = 20          # apply 8 + apply 8 + reduce 4
EXPR1 = "x = x*1.0001 + 0.5"
EXPR2 = "x = sqrt(x)"
L2_BYTES = 126 << 20


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smmax, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smmax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smmax) if smmax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# dram__bytes_read.sum + dram__bytes_write.sum of thb_apply_contig for 2^28 elements, per element
# (profiles/apply_contig_and_reduce_all_2p28.md); DRAM traffic of this kernel grows in proportion.
NCU_DRAM_BYTES_PER_ELT_APPLY = (1.073748e9 + 1.015486e9) / 268435456


# ---- CPU leg (oracle port) ---------------------------------------------------------------------

def cpu_chain(sample_elems: int, reps: int, threads: int = 0):
    """The same chain on the host cores with the oracle's fp32 loops; returns (GB/s, threads).
    threads = 0: every core this process may use."""
    import numpy as np
    from oracle import oracle as O
    L = O.lib()
    # torchrun exports OMP_NUM_THREADS=1 to its ranks: set the count explicitly
    L.orc_set_num_threads(threads if threads > 0 else len(os.sched_getaffinity(0)))
    g = np.random.Generator(np.random.PCG64(4))
    x = g.random(sample_elems, dtype=np.float32)
    ptr = C.c_void_p(x.ctypes.data)
    L.orc_time_axpb(ptr, sample_elems, 1.0001, 0.5)      # touch / warm
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        L.orc_time_axpb(ptr, sample_elems, 1.0001, 0.5)
        L.orc_time_sqrt(ptr, sample_elems)
        L.orc_time_sum(ptr, sample_elems)
        times.append(time.perf_counter() - t0)
    return BYTES_PER_ELT * sample_elems / statistics.median(times) / 1e9, L.orc_num_threads()


def torch_cpu_chain(sample_elems: int, reps: int):
    """A second, independent CPU number: the same chain with PyTorch's CPU kernels on all cores."""
    import numpy as np
    import torch
    threads = len(os.sched_getaffinity(0))
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
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 1 << 27
    per_step = []
    threads = 1
    for _ in range(args.warmup):
        cpu_chain(sample, 1)
    for _ in range(args.steps):
        gbs, threads = cpu_chain(sample, 3)
        per_step.append(gbs)
    value = statistics.median(per_step)
    line = {
        "impl": "reference", "metric": "achieved_hbm_gbs_sharded_apply_reduceall", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": BYTES_PER_ELT * sample / value / 1e6, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c5_sharded_apply_reduceall", "elements": N_TOTAL, "sample_elements": sample,
                   "note": "CPU restatement of the reference path (the reference needs OpenCL + Torch7, absent here)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"2^27 of the 2^31 elements, 3 repetitions per step, OpenMP on {threads} threads"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- GPU leg -------------------------------------------------------------------------------------

def run_gpu(args):
    import numpy as np
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

    gsum = GlobalSum()                      # binds the library to this GPU and to torch's current stream
    n_total = args.elements
    begin, end = shard_bounds(n_total, world, rank)
    n_local = end - begin

    # shard in pinned host memory (for e2e) and resident on the device (for value)
    host = torch.empty(n_local, dtype=torch.float32, pin_memory=True)
    hview = host.numpy()
    g = np.random.Generator(np.random.PCG64(4).jumped(rank))
    chunk = 1 << 26
    for s in range(0, n_local, chunk):
        e = min(n_local, s + chunk)
        hview[s:e] = g.random(e - s, dtype=np.float32)
    x = cl.ClTensor(n_local)
    x.copy(hview)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step(events=None):
        if events is not None:
            events[0].record()
        x.apply_on_gpu(EXPR1)
        if events is not None:
            events[1].record()
        x.apply_on_gpu(EXPR2)
        if events is not None:
            events[2].record()
        r = gsum(x)
        if events is not None:
            events[3].record()
        return r

    # nvidia-smi needs a few hundred ms to deliver its first samples: start it before the
    # warm-up and keep the GPU busy for at least half a second before the timed region
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
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
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = start.elapsed_time(stop)
    total_gpu = float(result.s())

    # e2e: host buffer -> device, chain, result back to the host; every step
    e2e_steps = args.steps
    for _ in range(2):
        x.copy(hview); step().s()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        x.copy(hview)
        total_e2e = step().s()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    times = torch.tensor([elapsed_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = times.tolist()

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = elapsed_ms / args.steps
        value = BYTES_PER_ELT * n_total / (ms_per_step * 1e-3) / 1e9
        k_apply = statistics.mean(e[0].elapsed_time(e[1]) for e in step_events)
        k_apply2 = statistics.mean(e[1].elapsed_time(e[2]) for e in step_events)
        k_sum = statistics.mean(e[2].elapsed_time(e[3]) for e in step_events)
        achieved = 8 * n_local / (k_apply * 1e-3) / 1e9
        line = {
            "metric": "achieved_hbm_gbs_sharded_apply_reduceall", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "c5_sharded_apply_reduceall", "elements": n_total, "elements_per_gpu": n_local,
                       "extra_untimed_warmup_steps": args.clock_warmup * world,
                       "ops": [EXPR1, EXPR2, "sum (reduceAll) + all-gather of 1 float per GPU + fixed-order fold"],
                       "algorithmic_bytes_per_element": BYTES_PER_ELT, "parallelism": f"shard{world}",
                       "l2": f"inputs larger than L2 ({4 * n_local >> 20} MiB per GPU vs 126 MiB)"},
            "roofline": {"bound": "hbm", "kernel": "thb_apply_contig<UserOp,1> (x = x*1.0001 + 0.5)",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "traffic": NCU_DRAM_BYTES_PER_ELT_APPLY * n_local,
                         "traffic_note": "bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu "
                                         "capture at 2^28 elements (2.0892 GB), scaled by the elements of a launch",
                         "per_kernel_gbs": {"apply_axpb": achieved, "apply_sqrt": 8 * n_local / (k_apply2 * 1e-3) / 1e9,
                                            "reduce_all_sum": 4 * n_local / (k_sum * 1e-3) / 1e9}},
            "e2e": {"value": BYTES_PER_ELT * n_total / (e2e_ms / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": 4 * n_local, "d2h_bytes_per_step": 4, "steps": e2e_steps},
            "gpu_launches": args.steps * (2 + gsum.launches_per_call),
            "clocks": clocks, "check": {"global_sum": total_gpu, "global_sum_e2e": float(total_e2e)},
        }
        if world == 1:
            gbs, threads = cpu_chain(1 << 27, 12)
            one, _ = cpu_chain(1 << 25, 3, threads=1)
            tgbs, tthreads = torch_cpu_chain(1 << 27, 5)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"2^27 of the 2^31 elements, median of 12 repetitions, OpenMP on {threads} threads",
                                    "one_thread": {"value": one, "unit": "GB/s", "cores": 1,
                                                   "sample": "2^25 elements, median of 3 repetitions"},
                                    "torch_cpu": {"value": tgbs, "unit": "GB/s", "cores": tthreads,
                                                  "sample": "2^27 elements, median of 5 repetitions, counted at the same "
                                                            "20 algorithmic bytes per element"}}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5")
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
        from cltorch_b200 import bench_configs
        bench_configs.run(args.workload, args.steps, max(args.warmup, 3))


if __name__ == "__main__":
    main()
