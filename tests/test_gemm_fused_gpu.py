"""thb200_gemm with the hi/lo split inside the kernel - both operands split in shared memory by one CTA per
tile ("fused") or by pairs of CTAs on 256-row tiles ("pair"), or A' split into tensor memory with only B'
pre-split ("ts") - against the same call with the split
pre-pass and against an fp64-accumulated CPU GEMM: every transposition pair, ragged edges, K not a multiple of the k block,
batches, split-K, alpha/beta. The library reads THB200_GEMM_MODE once per process, so each
path runs in a child process of its own (this file is also that child's program).

Tolerance: 1e-4 relative (Frobenius norm and worst element against the largest entry), as for
every GEMM test; the two paths round the operands identically and are expected to agree to ~1e-6.
"""
import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent

# (transa, transb, m, n, k, batch, alpha, beta); leading dimensions are padded to a multiple of 4
CASES = [
    ("n", "n", 128, 256, 64, 1, 1.0, 0.0),
    ("n", "n", 132, 260, 100, 1, 2.0, 0.5),
    ("t", "n", 132, 260, 100, 1, 1.0, 1.0),
    ("n", "t", 132, 260, 100, 1, 1.0, 1.0),
    ("t", "t", 132, 260, 100, 1, -1.0, 0.25),
    ("n", "n", 4, 8, 12, 1, 1.0, 0.0),
    ("t", "t", 36, 20, 7, 1, 1.0, 0.0),
    ("n", "n", 640, 512, 1000, 1, 1.0, 1.0),
    ("n", "n", 256, 256, 2048, 1, 1.0, 1.0),          # few tiles, long K: split along K
    ("t", "n", 300, 500, 4100, 1, 0.5, 2.0),
    ("n", "n", 256, 256, 128, 6, 1.0, 1.0),           # batched, short K
    ("n", "t", 200, 136, 48, 5, 1.0, 0.0),
    ("t", "n", 1024, 1024, 128, 3, 1.0, 1.0),
]


def _child(mode):
    sys.path.insert(0, str(ROOT))
    import cltorch_b200 as cl
    from cltorch_b200 import _lib
    L = cl.lib()
    cl.setDevice(1)
    stream = C.c_void_p(cl.getStream())
    out = {}
    for idx, (ta, tb, m, n, k, batch, alpha, beta) in enumerate(CASES):
        g = np.random.Generator(np.random.PCG64(900 + idx))
        # column-major storage: op(A) is m x k; 'n' stores m x k with lda >= m, 't' stores k x m with lda >= k
        ar, ac = (m, k) if ta == "n" else (k, m)
        br, bc = (k, n) if tb == "n" else (n, k)
        lda, ldb, ldc = (ar + 3) // 4 * 4 + 4, (br + 3) // 4 * 4, (m + 3) // 4 * 4
        a = g.uniform(-1, 1, (batch, ac, lda)).astype(np.float32)      # [batch][column][row within ld]
        b = g.uniform(-1, 1, (batch, bc, ldb)).astype(np.float32)
        c0 = g.uniform(-1, 1, (batch, n, ldc)).astype(np.float32)
        A, B, Cc = cl.ClTensor(a.reshape(-1)), cl.ClTensor(b.reshape(-1)), cl.ClTensor(c0.reshape(-1).copy())
        need = L.thb200_gemm_workspace_bytes(m, n, k, batch)
        ws = cl.ClStorage(need // 4 + 256)
        rc = L.thb200_gemm(stream, ta.encode(), tb.encode(), m, n, k, alpha, C.c_void_p(A.data_ptr()), lda,
                           C.c_void_p(B.data_ptr()), ldb, beta, C.c_void_p(Cc.data_ptr()), ldc, batch,
                           ac * lda, bc * ldb, n * ldc, C.c_void_p(ws.data_ptr()), C.c_size_t(ws.size() * 4))
        assert rc == 0, L.thb200_last_error()
        assert L.thb200_gemm_status(stream, m, n, k, batch, C.c_void_p(ws.data_ptr())) == 0
        got = Cc.float().reshape(batch, n, ldc)
        # a[b][col][row]: 'n' holds op(A)[i][kk] at a[b][kk][i]; 't' holds it at a[b][i][kk]
        opa = a[:, :k, :m].transpose(0, 2, 1) if ta == "n" else a[:, :m, :k]          # batch x m x k
        opb = b[:, :n, :k].transpose(0, 2, 1) if tb == "n" else b[:, :k, :n]          # batch x k x n
        want = beta * c0[:, :, :m].astype(np.float64).transpose(0, 2, 1) + alpha * np.einsum(
            "bik,bkj->bij", opa.astype(np.float64), opb.astype(np.float64))
        res = got[:, :, :m].transpose(0, 2, 1).astype(np.float64)
        err = np.linalg.norm(res - want) / max(np.linalg.norm(want), 1e-30)
        worst = np.abs(res - want).max() / (np.abs(want).max() + 1e-30)
        pad_untouched = bool(np.array_equal(got[:, :, m:], c0[:, :, m:]))
        out[str(idx)] = {"err": err, "worst": worst, "pad_untouched": pad_untouched,
                         "digest": float(np.sum(res * np.cos(np.arange(res.size).reshape(res.shape) % 97)))}
    print("RESULT " + json.dumps({"mode": mode, "cases": out}))


def _run(mode):
    env = dict(os.environ, THB200_GEMM_MODE=mode)
    r = subprocess.run([sys.executable, __file__, mode], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])["cases"]


@pytest.mark.gpu
def test_split_inside_the_kernels_matches_prepass_and_fp64():
    prepass = _run("prepass")
    bad = []
    for mode in ("fused", "ts", "pair"):
        res = _run(mode)
        for idx, case in enumerate(CASES):
            f, p = res[str(idx)], prepass[str(idx)]
            if not (f["err"] <= 1e-4 and f["worst"] <= 1e-4):
                bad.append((mode, case, f))
            if mode == "fused" and not (p["err"] <= 1e-4 and p["worst"] <= 1e-4):
                bad.append(("prepass", case, p))
            if not (f["pad_untouched"] and p["pad_untouched"]):                  # nothing written between m and ldc
                bad.append((mode, "padding written", case, f, p))
            if abs(f["digest"] - p["digest"]) > 1e-4 * (abs(p["digest"]) + 1.0):
                bad.append((mode, "paths disagree", case, f["digest"], p["digest"]))
    assert not bad, "\n".join(str(b) for b in bad)


if __name__ == "__main__":
    _child(sys.argv[1])
