"""Per-operation timings of benchmark configurations 1-4 on one GPU.

`bench.py` runs the groups c1..c4 after its default workload and puts them into its JSON line;
`bench.py --workload NAME` runs one group alone (also the smaller `c2small|c3small|c4small|
c4batched|n3small` shapes that profiler captures use, and the `n1|n3` operation tables).

Every operation is timed on its own with CUDA events on the stream the library launches on:
median of at least `steps` calls after `warmup` calls, repeated until the GPU has been busy for
a quarter of a second so that clock samples exist for the group. Rates use the ALGORITHMIC bytes
(4 bytes per element an operation must read or write) or 2*M*N*K flops, and are quoted against
the measured HBM copy rate (MEASURED_PEAKS.json) or, for the GEMM, against one third of the
dense TF32 rate (three TF32 products per fp32 product): the nominal 1100 TFLOP/s and the
single-pass TF32 rate of the library GEMM measured in the same run.
Inputs are seeded synthetic tensors of the configured shapes. Each group carries its own
clock record (nvidia-smi samples taken while the group's timed calls ran).
"""
from __future__ import annotations

import datetime
import json
import statistics
import subprocess
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
TF32_DENSE_TFLOPS_NOMINAL = 1100.0
MIN_BUSY_S = 0.25
MAX_CALLS = 4000


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples with time stamps (read-only queries).

    One process samples every 100 ms for the whole run; `summary(windows)` reduces the samples that
    fall inside the given wall-clock windows, so each group of timed calls gets its own record.
    """

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.samples = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def stop(self):
        """Ends the sampling process and parses what it printed."""
        if self.samples is not None:
            return
        self.samples = []
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sm, smmax, power = float(f[2]), float(f[3]), float(f[4])
            except ValueError:
                continue
            active = {name for name, val in zip(self.REASONS, f[6:10]) if val.lower().startswith("active")}
            self.samples.append((ts, sm, smmax, power, active))

    def summary(self, windows=None):
        """Median SM clock, maximum clock, power and throttle reasons over the samples inside `windows`
        (a list of (t0, t1) wall-clock pairs; None = every sample)."""
        self.stop()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        pick = [s for s in self.samples
                if windows is None or any(t0 <= s[0] <= t1 for t0, t1 in windows)]
        reasons = set()
        for s in pick:
            reasons |= s[4]
        return {"sm_mhz": statistics.median(s[1] for s in pick) if pick else None,
                "sm_max_mhz": max(s[2] for s in pick) if pick else None,
                "power_w_max": max(s[3] for s in pick) if pick else None,
                "samples": len(pick), "reasons": sorted(reasons)}


class Timer:
    def __init__(self, steps, warmup, sampler=None):
        import torch
        import cltorch_b200 as cl
        self.torch, self.cl = torch, cl
        torch.cuda.set_device(0)
        cl.setDevice(1)
        cl.setStream(torch.cuda.current_stream().cuda_stream)
        self.steps, self.warmup = steps, warmup
        self.flush = torch.empty(128 << 20, dtype=torch.float32, device="cuda")
        self.flush_read = torch.zeros(64 << 20, dtype=torch.float32, device="cuda")
        self.peak = measured_peaks()["hbm_gbs"]
        self.sampler = sampler
        self.results = {}
        self.windows = []
        self.launch_calls = 0

    def take_group(self):
        """Results and clock windows collected since the last call, as one group record."""
        res, win = self.results, self.windows
        self.results, self.windows = {}, []
        return res, win

    def _flush_l2(self, clean):
        self.flush.fill_(1.0)
        if clean:
            self.flush_read.sum()

    def time(self, name, fn, nbytes=None, flops=None, setup=None, also_dirty=False):
        """Median CUDA-event time of fn() over at least `steps` calls after `warmup` calls.

        L2 state: a call that moves at least 1 GiB works on operands of 512 MiB or more (four times
        the 126 MB L2) and runs back to back on them: every read is cold because the operands evict
        themselves, and the dirty lines a call finds in L2 are the previous call's own output, as in
        steady state. Smaller calls are preceded by a 512 MiB fill that evicts their operands and a
        256 MiB read that pushes the fill's dirty lines out, so the call starts with L2 cold and
        clean. `also_dirty` adds the time after the fill alone (`ms_after_fill_only`): up to 126 MB
        of dirty lines are then written back while the call runs, which is a lower bound for it.
        """
        t = self.torch
        flush = nbytes is None or nbytes < (1 << 30)

        def run(clean):
            ms = []
            w0 = time.time()
            while len(ms) < self.steps or (time.time() - w0 < MIN_BUSY_S and len(ms) < MAX_CALLS):
                if setup:
                    setup()
                if flush:
                    self._flush_l2(clean)
                a, b = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                b.synchronize()
                ms.append(a.elapsed_time(b))
            self.windows.append((w0, time.time()))
            self.launch_calls += len(ms)
            return ms

        for _ in range(self.warmup):
            if setup:
                setup()
            fn()
        ms = run(True)
        med = statistics.median(ms)
        r = {"ms": med, "calls": len(ms),
             "l2": "512 MiB fill and 256 MiB read before each call (cold, clean L2)" if flush
             else "operands >= 4 x L2, calls back to back"}
        if also_dirty and flush:
            r["ms_after_fill_only"] = statistics.median(run(False))
        if nbytes is not None:
            r["bytes"] = nbytes
            r["GB/s"] = nbytes / (med * 1e-3) / 1e9
            r["frac_of_measured_hbm"] = r["GB/s"] / self.peak
            r["frac_of_nominal_8TBs"] = r["GB/s"] / 8000.0
        if flops is not None:
            r["flops"] = flops
            r["TFLOP/s"] = flops / (med * 1e-3) / 1e12
            r["frac_of_3xtf32_nominal"] = r["TFLOP/s"] / (TF32_DENSE_TFLOPS_NOMINAL / 3)
        self.results[name] = r
        return r


def _uniform(g, shape, lo, hi):
    return (g.random(shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def c1(T):
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(0))
    n = 4096 * 4096
    X, Y, Z = (cl.ClTensor(_uniform(g, (4096, 4096), 0, 1)) for _ in range(3))
    S = cl.ClTensor()
    one = cl.ClTensor(1)
    T.time("timing floor: fill of a 1-element tensor (launch + the two event records)", lambda: one.fill(0.0))
    T.time("map2 x = sqrt(1000*x + y*10 + z*z)", lambda: X.map2_on_gpu(Y, Z, "x = sqrt(1000*x + y*10 + z*z)"), 16 * n,
           also_dirty=True)
    T.time("sum -> point tensor", lambda: S.sum(X), 4 * n, also_dirty=True)
    T.time("div by point tensor", lambda: X.div(S), 8 * n, setup=lambda: X.fill(1.0) and S.sum(X), also_dirty=True)
    T.time("sum -> host float (with read-back)", lambda: X.sum(), 4 * n, also_dirty=True)
    T.time("div by host float", lambda: X.div(3.0), 8 * n)

    def chain():
        X.map2_on_gpu(Y, Z, "x = sqrt(1000*x + y*10 + z*z)")
        S.sum(X)
        X.div(S)
    T.time("sequence map2 + sum + div (point tensor)", chain, 28 * n, also_dirty=True)

    def chain_host():
        X.map2_on_gpu(Y, Z, "x = sqrt(1000*x + y*10 + z*z)")
        X.div(X.sum())
    T.time("sequence map2 + s = sum (host float) + div(s), as the configuration is worded", chain_host, 28 * n)

    # The same operations in steady state: eight sets of tensors (1.5 GiB, twelve times L2) taken in
    # turn and launched back to back, so every operand comes from HBM and the launch and event
    # overheads of the single calls above (the timing floor) are spread over eight calls.
    sets = [(X, Y, Z)] + [tuple(cl.ClTensor(_uniform(g, (4096, 4096), 0, 1)) for _ in range(3)) for _ in range(7)]
    pts = [cl.ClTensor() for _ in range(8)]
    T.time("8 x map2 on eight tensor sets, back to back", lambda: [x.map2_on_gpu(y, z, "x = sqrt(1000*x + y*10 + z*z)") for x, y, z in sets],
           8 * 16 * n)
    T.time("8 x sum -> point tensor on eight tensors, back to back", lambda: [p.sum(s[0]) for p, s in zip(pts, sets)], 8 * 4 * n)
    T.time("8 x div by point tensor on eight tensors, back to back", lambda: [s[0].div(p) for p, s in zip(pts, sets)], 8 * 8 * n,
           setup=lambda: [s[0].fill(1.0) and p.sum(s[0]) for p, s in zip(pts, sets)])

    def chains():
        for p, (x, y, z) in zip(pts, sets):
            x.map2_on_gpu(y, z, "x = sqrt(1000*x + y*10 + z*z)")
            p.sum(x)
            x.div(p)
    T.time("8 x sequence map2 + sum + div (point tensor), back to back", chains, 8 * 28 * n)


def c2(T):
    cl = T.cl
    n = 8192
    g = np.random.Generator(np.random.PCG64(1))
    A, B, Tt = (cl.ClTensor(_uniform(g, (n, n), -1, 1)) for _ in range(3))
    views = {
        "T (transpose)": lambda X: X.t(),
        "S (stride-2 columns)": lambda X: cl.ClTensor(X.storage(), 1, [n, n // 2], [n, 2]),
        "W (narrow rows)": lambda X: X.narrow(1, 17, 4000),
        "Wc (narrow columns)": lambda X: X.narrow(2, 17, 4000),
    }
    for name, gv in views.items():
        va, vb, vt = gv(A), gv(B), gv(Tt)
        cnt = va.nElement()
        out = cl.ClTensor().resizeAs(va)
        T.time(f"add {name}", lambda: out.add(va, vb), 12 * cnt)
        T.time(f"cmul {name}", lambda: out.cmul(va, vb), 12 * cnt)
        T.time(f"addcmul(0.5) {name} [copy + apply3 = 24 B/elt]", lambda: out.addcmul(vt, 0.5, va, vb), 24 * cnt)
        T.time(f"copy into fresh contiguous {name}", lambda: out.copy(va), 8 * cnt)
        T.time(f"apply x = tanh(x)*x (in place, contiguous copy) {name}", lambda: out.apply_on_gpu("x = tanh(x)*x"), 8 * cnt,
               setup=lambda: out.copy(va))
    out = cl.ClTensor(n, n)
    T.time("add contiguous = transpose + contiguous", lambda: out.add(A.t(), B), 12 * n * n)


def c3(T):
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(2))
    a = g.standard_normal((16384, 16384), dtype=np.float32)
    A = cl.ClTensor(a)
    del a
    n = 16384 * 16384
    out = cl.ClTensor()
    for d in (1, 2):
        T.time(f"sum(A, {d})", lambda: out.sum(A, d), 4 * n)
        T.time(f"max(A, {d}) with indices", lambda: A.max(d), 4 * n)
        T.time(f"min(A, {d}) with indices", lambda: A.min(d), 4 * n)
    m, s = cl.ClTensor(), cl.ClTensor()

    def chain():
        for _ in range(100):
            m.mean(A); A.csub(m); s.std(A); A.div(s)
    T.time("100 x (mean, sub, std, div) on the device [24 B/elt per iteration: std is one pass]", chain, 100 * 24 * n)
    del A
    b = g.standard_normal((256, 1024, 1024), dtype=np.float32)
    Bt = cl.ClTensor(b)
    del b
    for d in (1, 2, 3):
        T.time(f"sum(B3d, {d})", lambda: out.sum(Bt, d), 4 * n)
        T.time(f"max(B3d, {d}) with indices", lambda: Bt.max(d), 4 * n)
        T.time(f"min(B3d, {d}) with indices", lambda: Bt.min(d), 4 * n)


def library_tf32_rate(T):
    """Library reference points on the same box and stream: the single-pass TF32 GEMM (the tensor
    pipe's measured ceiling; a 3xTF32 GEMM can reach at most a third of it) and the fp32 GEMM.
    Returns the TF32 rate in TFLOP/s, or None where this torch build lacks the switches."""
    t = T.torch
    try:
        ta = t.rand(8192, 8192, device="cuda") - 0.5
        tb = t.rand(8192, 8192, device="cuda") - 0.5
        tc = t.empty(8192, 8192, device="cuda")
        was = t.backends.cuda.matmul.allow_tf32
        t.backends.cuda.matmul.allow_tf32 = True
        r = T.time("library: single-pass TF32 GEMM 8192x8192x8192", lambda: t.matmul(ta, tb, out=tc), flops=2.0 * 8192 ** 3)
        r["third_of_measured_tf32_TFLOP/s"] = r["TFLOP/s"] / 3
        t.backends.cuda.matmul.allow_tf32 = False
        T.time("library: fp32 GEMM 8192x8192x8192", lambda: t.matmul(ta, tb, out=tc), flops=2.0 * 8192 ** 3)
        t.backends.cuda.matmul.allow_tf32 = was
        for k in ("library: single-pass TF32 GEMM 8192x8192x8192", "library: fp32 GEMM 8192x8192x8192"):
            T.results[k].pop("frac_of_3xtf32_nominal", None)
        return r["TFLOP/s"]
    except Exception as e:  # the library points are optional
        T.results["library reference points"] = {"ms": 0.0, "error": str(e)[:200]}
        return None


def c4(T):
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(3))
    tf32 = library_tf32_rate(T)

    def pair(M, N, K, batch=None):
        lim = 1.0 / np.sqrt(K)
        sa = (M, K) if batch is None else (batch, M, K)
        sb = (K, N) if batch is None else (batch, K, N)
        return cl.ClTensor(_uniform(g, sa, -lim, lim)), cl.ClTensor(_uniform(g, sb, -lim, lim))

    def third(r):
        if tf32:
            r["frac_of_third_of_measured_tf32"] = r["TFLOP/s"] / (tf32 / 3)

    for M, N, K in ((8192, 8192, 8192), (512, 4096, 4096)):
        A, B = pair(M, N, K)
        C = cl.ClTensor(M, N).zero()
        third(T.time(f"addmm {M}x{N}x{K}", lambda: C.addmm(1.0, C, 1.0, A, B), flops=2.0 * M * N * K, setup=lambda: C.zero()))
        del A, B, C
    A, B = pair(1024, 1024, 128, batch=64)
    C = cl.ClTensor(64, 1024, 1024).zero()
    nbytes = 64 * (1024 * 128 + 128 * 1024 + 2 * 1024 * 1024) * 4
    third(T.time("baddbmm 64 x (1024x1024x128)", lambda: C.baddbmm(1.0, C, 1.0, A, B), nbytes=nbytes,
                 flops=2.0 * 64 * 1024 * 1024 * 128, setup=lambda: C.zero()))


def c4batched(T):
    """The batched K = 128 shape alone, with and without the read of C (profiler captures, experiments)."""
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(3))
    lim = 1.0 / np.sqrt(128)
    A = cl.ClTensor(_uniform(g, (64, 1024, 128), -lim, lim))
    B = cl.ClTensor(_uniform(g, (64, 128, 1024), -lim, lim))
    C = cl.ClTensor(64, 1024, 1024).zero()
    flops = 2.0 * 64 * 1024 * 1024 * 128
    T.time("baddbmm 64 x (1024x1024x128), beta = 1", lambda: C.baddbmm(1.0, C, 1.0, A, B),
           nbytes=64 * (1024 * 128 + 128 * 1024 + 2 * 1024 * 1024) * 4, flops=flops, setup=lambda: C.zero())
    T.time("bmm 64 x (1024x1024x128), beta = 0", lambda: C.bmm(A, B),
           nbytes=64 * (1024 * 128 + 128 * 1024 + 1024 * 1024) * 4, flops=flops)


def c4small(T):
    """One mid-sized addmm (2048 x 2048 x 4096): the case used for profiler captures of the GEMM kernels."""
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(3))
    M, N, K = 2048, 2048, 4096
    lim = 1.0 / np.sqrt(K)
    A, B = cl.ClTensor(_uniform(g, (M, K), -lim, lim)), cl.ClTensor(_uniform(g, (K, N), -lim, lim))
    C = cl.ClTensor(M, N).zero()
    T.time(f"addmm {M}x{N}x{K}", lambda: C.addmm(1.0, C, 1.0, A, B), flops=2.0 * M * N * K, setup=lambda: C.zero())


def c4mlp(T):
    """The 512 x 4096 x 4096 addmm alone (profiler captures of the tensor-memory GEMM and the split-K fix-up)."""
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(3))
    M, N, K = 512, 4096, 4096
    lim = 1.0 / np.sqrt(K)
    A, B = cl.ClTensor(_uniform(g, (M, K), -lim, lim)), cl.ClTensor(_uniform(g, (K, N), -lim, lim))
    C = cl.ClTensor(M, N).zero()
    T.time(f"addmm {M}x{N}x{K}", lambda: C.addmm(1.0, C, 1.0, A, B), flops=2.0 * M * N * K, setup=lambda: C.zero())


def c2small(T):
    """Transpose and column-narrowed adds on 4096 x 4096 (profiler captures of the strided kernels)."""
    cl = T.cl
    n = 4096
    g = np.random.Generator(np.random.PCG64(1))
    A, B = (cl.ClTensor(_uniform(g, (n, n), -1, 1)) for _ in range(2))
    out = cl.ClTensor(n, n)
    T.time("add contiguous = transpose + transpose", lambda: out.add(A.t(), B.t()), 12 * n * n)
    va, vb = A.narrow(2, 17, 2000), B.narrow(2, 17, 2000)
    out2 = cl.ClTensor().resizeAs(va)
    T.time("add narrow-columns", lambda: out2.add(va, vb), 12 * n * 2000)


def c3small(T):
    """Sums and max-with-indices along both dimensions of 8192 x 8192 (profiler captures of the reductions)."""
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(2))
    n = 8192
    A = cl.ClTensor(g.standard_normal((n, n), dtype=np.float32))
    out = cl.ClTensor()
    for d in (1, 2):
        T.time(f"sum(A, {d})", lambda: out.sum(A, d), 4 * n * n)
        T.time(f"max(A, {d}) with indices", lambda: A.max(d), 4 * n * n)


def n3(T):
    """var/std along a dimension, scans, renorm and dist on 16384 x 16384 (1 GiB)."""
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(5))
    rows = 16384
    n = rows * rows
    a = g.standard_normal((rows, rows), dtype=np.float32)
    A = cl.ClTensor(a)
    del a
    out = cl.ClTensor()
    for d in (1, 2):
        T.time(f"var(A, {d})", lambda: out.var(A, d), 4 * n)
        T.time(f"std(A, {d}, true)", lambda: out.std(A, d, True), 4 * n)
    pt = cl.ClTensor()
    T.time("std -> point tensor (one pass)", lambda: pt.std(A), 4 * n)
    T.time("norm(2) -> host float", lambda: A.norm(2), 4 * n)
    T.time("norm(3) -> host float", lambda: A.norm(3), 4 * n)
    T.time("norm(2.5) -> host float [general power: exp2(p*log2|x|) per element]", lambda: A.norm(2.5), 4 * n)
    B = cl.ClTensor(rows, rows)
    for d in (1, 2):
        T.time(f"cumsum(A, {d}) [8 B/elt; the chunked form moves 12]", lambda: B.cumsum(A, d), 8 * n)
    T.time("cumprod(A, 2)", lambda: B.cumprod(A, 2), 8 * n)
    V = cl.ClTensor(g.standard_normal((n,), dtype=np.float32))
    W = cl.ClTensor(n)
    T.time("cumsum of a 2^28 vector [8 B/elt; single pass, tiles wait for their carries in L2]", lambda: W.cumsum(V, 1), 8 * n)
    T.time("dist(A, B, 2) -> point tensor", lambda: pt.dist_gpu(A, B, 2), 8 * n)
    # renorm in place along dimension 1 (rows of 16384 normal values have 2-norms close to 128:
    # about half of them exceed the limit and are rescaled); A is restored before every call
    A0 = cl.ClTensor(rows, rows).copy(A)
    T.time("renorm(A, 2, 1, 128) in place [one pass: 4 B/elt read + 4 B/elt written for the half of the rows rescaled]",
           lambda: A.renorm(A, 2, 1, 128.0), 4 * n + 2 * n, setup=lambda: A.copy(A0))


def n1(T):
    """dot, addmv (both orientations of the matrix) and addr on 16384 x 16384 / 2^28 elements."""
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(6))
    n = 16384
    M = cl.ClTensor(_uniform(g, (n, n), -1, 1))
    x = cl.ClTensor(_uniform(g, (n,), -1, 1))
    y = cl.ClTensor(n).zero()
    T.time("addmv y = y + M x (row-major M)", lambda: y.addmv(1.0, 1.0, M, x), 4 * n * n, setup=lambda: y.zero())
    Mt = M.t()
    T.time("addmv y = y + M^T x (transposed view)", lambda: y.addmv(1.0, 1.0, Mt, x), 4 * n * n, setup=lambda: y.zero())
    R = cl.ClTensor(n, n).zero()
    T.time("addr R = R + x (x) x [8 B/elt]", lambda: R.addr(1.0, x, x), 8 * n * n)
    a = cl.ClTensor(_uniform(g, (n * n,), -1, 1))
    b = cl.ClTensor(_uniform(g, (n * n,), -1, 1))
    T.time("dot of two 2^28 vectors -> host float [8 B/elt]", lambda: a.dot(b), 8 * n * n)


def n3small(T):
    """var, cumsum, dist and renorm on 8192 x 8192 and cumsum of a 2^26 vector (profiler captures of the moments, scan and renorm kernels)."""
    cl = T.cl
    g = np.random.Generator(np.random.PCG64(5))
    n = 8192
    A = cl.ClTensor(g.standard_normal((n, n), dtype=np.float32))
    B = cl.ClTensor(n, n)
    out, pt = cl.ClTensor(), cl.ClTensor()
    for d in (1, 2):
        T.time(f"var(A, {d})", lambda: out.var(A, d), 4 * n * n)
        T.time(f"cumsum(A, {d})", lambda: B.cumsum(A, d), 8 * n * n)
    T.time("dist(A, B, 2) -> point tensor", lambda: pt.dist_gpu(A, B, 2), 8 * n * n)
    V = cl.ClTensor(g.standard_normal((1 << 26,), dtype=np.float32))
    W = cl.ClTensor(1 << 26)
    T.time("cumsum of a 2^26 vector", lambda: W.cumsum(V, 1), 8 << 26)
    # rows of 8192 standard-normal values have 2-norms close to 90.5: about half of them are rescaled
    A0 = cl.ClTensor(n, n).copy(A)
    T.time("renorm(A, 2, 1, 90.5) in place [4 B/elt read + 4 B/elt written for the rows rescaled]",
           lambda: A.renorm(A, 2, 1, 90.5), 4 * n * n + 2 * n * n, setup=lambda: A.copy(A0))


GROUPS = {"c1": c1, "c2": c2, "c3": c3, "c4": c4, "c4small": c4small, "c4batched": c4batched, "c4mlp": c4mlp, "c2small": c2small,
          "c3small": c3small, "n1": n1, "n3": n3, "n3small": n3small}


def run_groups(names, steps, warmup, sampler):
    """Runs the named groups one after the other; returns {name: {"results", "clocks", "launch_calls"}}.
    The sampler must be running; it is stopped here, after the last group."""
    T = Timer(steps, warmup, sampler)
    raw = {}
    for name in names:
        before = T.launch_calls
        GROUPS[name](T)
        T.cl.synchronize()
        res, win = T.take_group()
        raw[name] = (res, win, T.launch_calls - before)
        import gc
        gc.collect()
    out = {}
    for name, (res, win, calls) in raw.items():
        out[name] = {"results": res, "clocks": sampler.summary(win) if sampler else None, "timed_calls": calls}
    return out


def run(workload: str, steps: int, warmup: int) -> None:
    sampler = ClockSampler(0).start()
    groups = run_groups([workload], steps, warmup, sampler)
    print(json.dumps({"workload": workload, "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "f32",
                      "data": "synthetic", "hbm_peak_gbs_measured": measured_peaks()["hbm_gbs"],
                      "l2_flush": "per result: 512 MiB fill + 256 MiB read before each call, or none when a call moves "
                                  ">= 1 GiB (operands >= 4 x L2)",
                      "results": groups[workload]["results"], "clocks": groups[workload]["clocks"]}))
