"""The five benchmark workloads at their full sizes, checked for parity.

Inputs are seeded synthetic tensors (numpy PCG64), the same arrays for the GPU path and
for the CPU evaluation. Where a full CPU evaluation would take minutes, the check uses
properties that do not depend on the size: samples of rows, linearity (sum of a product
against the product of sums) and streaming double-precision sums.
"""
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def pcg(seed):
    return np.random.Generator(np.random.PCG64(seed))


def uniform(g, shape, lo, hi):
    return (g.random(shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def test_config1_map2_sum_div():
    """x:map2_on_gpu(y, z, "x = sqrt(1000*x + y*10 + z*z)"); s = x:sum(); x:div(s) on 4096 x 4096."""
    import cltorch_b200 as cl
    g = pcg(0)
    x, y, z = (uniform(g, (4096, 4096), 0, 1) for _ in range(3))
    X, Y, Z = cl.ClTensor(x), cl.ClTensor(y), cl.ClTensor(z)
    X.map2_on_gpu(Y, Z, "x = sqrt(1000*x + y*10 + z*z)")
    want = O.eval_expr("x = sqrt(1000*x + y*10 + z*z)", x, y, z)
    got = X.float()
    assert O.ulp_diff(got, want).max() <= 2
    assert np.array_equal(got, want)          # + * sqrt are exactly rounded on both sides
    total = float(want.astype(np.float64).sum())
    s = X.sum()
    assert abs(s - total) <= 1e-5 * total
    # host-scalar form: multiply by 1.0f / s
    X1 = cl.ClTensor(want).div(s)
    assert O.ulp_diff(X1.float(), want * (np.float32(1.0) / np.float32(s))).max() <= 2
    # point-tensor form: true division, nothing returns to the host in between
    S = cl.ClTensor()
    S.sum(X)
    X.div(S)
    assert abs(S.s() - total) <= 1e-5 * total
    assert O.ulp_diff(X.float(), want / np.float32(S.s())).max() <= 2


def test_config2_strided_apply():
    """Transpose view, stride-2 column slice and narrow views of 8192 x 8192 bases; results into fresh tensors."""
    import cltorch_b200 as cl
    n = 8192
    g = pcg(1)
    a, b, t = (uniform(g, (n, n), -1, 1) for _ in range(3))
    A, B, T = cl.ClTensor(a), cl.ClTensor(b), cl.ClTensor(t)
    views = {
        "T": (lambda X: X.t(), lambda v: v.T),
        "S": (lambda X: cl.ClTensor(X.storage(), 1, [n, n // 2], [n, 2]), lambda v: v[:, ::2]),
        "W": (lambda X: X.narrow(1, 17, 4000), lambda v: v[16:4016]),
        "Wc": (lambda X: X.narrow(2, 17, 4000), lambda v: v[:, 16:4016]),
    }
    for name, (gv, hv) in views.items():
        va, vb, vt = gv(A), gv(B), gv(T)
        ha, hb, ht = hv(a), hv(b), hv(t)
        out = cl.ClTensor()
        out.add(va, vb)
        assert out.isContiguous() and np.array_equal(out.float(), ha + hb), f"add {name}"
        out = cl.ClTensor()
        out.cmul(va, vb)
        assert np.array_equal(out.float(), ha * hb), f"cmul {name}"
        out = cl.ClTensor()
        out.addcmul(vt, 0.5, va, vb)
        assert np.array_equal(out.float(), ht + (np.float32(0.5) * ha) * hb), f"addcmul {name}"
        out = va.clone().apply_on_gpu("x = tanh(x)*x")
        want = np.tanh(ha.astype(np.float64)).astype(np.float32) * ha
        d = O.ulp_diff(out.float(), want)
        assert d.max() <= 2, f"tanh(x)*x {name}: {int(d.max())} ulp"
    # a mixed case: contiguous = transposed + contiguous
    out = cl.ClTensor()
    out.add(A.t(), B)
    assert np.array_equal(out.float(), a.T + b)


def test_config3_dim_reductions_and_device_chain():
    import cltorch_b200 as cl
    g = pcg(2)
    a = g.standard_normal((16384, 16384), dtype=np.float32)
    A = cl.ClTensor(a)
    for d in (0, 1):
        want = a.sum(axis=d, dtype=np.float64, keepdims=True)
        got = A.sum(d + 1).float()
        scale = np.abs(a).sum(axis=d, dtype=np.float64, keepdims=True)
        assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1e-3 * scale)), f"sum dim {d}"
        for name, fn, arg in (("max", np.max, np.argmax), ("min", np.min, np.argmin)):
            v, i = getattr(A, name)(d + 1)
            assert np.array_equal(v.float().squeeze(d), fn(a, axis=d)), f"{name} dim {d}"
            assert np.array_equal(i.long().squeeze(d), arg(a, axis=d) + 1), f"arg{name} dim {d}"
    # dependent chain, kept on the device through point tensors
    m, s = cl.ClTensor(), cl.ClTensor()
    for _ in range(100):
        m.mean(A); A.csub(m); s.std(A); A.div(s)
    out = A.float()
    assert abs(out.mean(dtype=np.float64)) < 1e-5
    assert abs(out.std(dtype=np.float64, ddof=1) - 1.0) < 1e-5
    ref = (a.astype(np.float64) - a.mean(dtype=np.float64)) / a.std(dtype=np.float64, ddof=1)
    assert np.abs(out[:64] - ref[:64]).max() < 1e-4       # 100 renormalisations leave the data where one put it
    del A, a, out, ref

    b = g.standard_normal((256, 1024, 1024), dtype=np.float32)
    B = cl.ClTensor(b)
    for d in (0, 1, 2):
        want = b.sum(axis=d, dtype=np.float64, keepdims=True)
        got = B.sum(d + 1).float()
        scale = np.abs(b).sum(axis=d, dtype=np.float64, keepdims=True)
        assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1e-3 * scale)), f"3-D sum dim {d}"
        v, i = B.max(d + 1)
        assert np.array_equal(v.float().squeeze(d), b.max(axis=d)), f"3-D max dim {d}"
        assert np.array_equal(i.long().squeeze(d), b.argmax(axis=d) + 1), f"3-D argmax dim {d}"
        v, i = B.min(d + 1)
        assert np.array_equal(i.long().squeeze(d), b.argmin(axis=d) + 1), f"3-D argmin dim {d}"


def _gemm_inputs(seed_gen, M, N, K, batch=None):
    lim = 1.0 / np.sqrt(K)
    sa = (M, K) if batch is None else (batch, M, K)
    sb = (K, N) if batch is None else (batch, K, N)
    return uniform(seed_gen, sa, -lim, lim), uniform(seed_gen, sb, -lim, lim)


def test_config4_gemm():
    import cltorch_b200 as cl
    g = pcg(3)
    # 8192^3: sampled rows in fp64 plus the linearity checksum sum(C) = colsum(A) . rowsum(B)
    a, b = _gemm_inputs(g, 8192, 8192, 8192)
    C = cl.ClTensor(8192, 8192).zero()
    C.addmm(1.0, C, 1.0, cl.ClTensor(a), cl.ClTensor(b))
    c = C.float()
    rows = pcg(99).choice(8192, size=48, replace=False)
    want = a[rows].astype(np.float64) @ b.astype(np.float64)
    err = np.linalg.norm(c[rows] - want) / np.linalg.norm(want)
    assert err <= 1e-4, f"8192^3 sampled rows: {err:.3e}"
    checksum = a.sum(axis=0, dtype=np.float64) @ b.sum(axis=1, dtype=np.float64)
    total = c.sum(dtype=np.float64)
    norm1 = np.abs(a).sum(axis=0, dtype=np.float64) @ np.abs(b).sum(axis=1, dtype=np.float64)
    assert abs(total - checksum) <= 1e-5 * norm1, (total, checksum)
    del a, b, c, C
    # MLP shape, full fp64 check
    a, b = _gemm_inputs(g, 512, 4096, 4096)
    C = cl.ClTensor(512, 4096).zero()
    C.addmm(1.0, C, 1.0, cl.ClTensor(a), cl.ClTensor(b))
    want = a.astype(np.float64) @ b.astype(np.float64)
    err = np.linalg.norm(C.float() - want) / np.linalg.norm(want)
    assert err <= 1e-4, f"512x4096x4096: {err:.3e}"
    # batched 64 x (1024 x 1024 x 128)
    a, b = _gemm_inputs(g, 1024, 1024, 128, batch=64)
    C = cl.ClTensor(64, 1024, 1024).zero()
    C.baddbmm(1.0, C, 1.0, cl.ClTensor(a), cl.ClTensor(b))
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    err = np.linalg.norm(C.float() - want) / np.linalg.norm(want)
    assert err <= 1e-4, f"batched: {err:.3e}"


def test_config5_large_vector_chain_single_gpu():
    """2^31-element vector: x = x*1.0001 + 0.5; x = sqrt(x); sum. Filled and checked in chunks."""
    import cltorch_b200 as cl
    n, chunk = 1 << 31, 1 << 26
    X = cl.ClTensor(n)
    g = pcg(4)
    total = 0.0
    probe = None
    for c in range(n // chunk):
        h = g.random(chunk, dtype=np.float32)
        X.narrow(1, c * chunk + 1, chunk).copy(h)
        w = np.sqrt(h * np.float32(1.0001) + np.float32(0.5))
        total += float(w.sum(dtype=np.float64))
        if c == 17:
            probe = w
    X.apply_on_gpu("x = x*1.0001 + 0.5")
    X.apply_on_gpu("x = sqrt(x)")
    S = cl.ClTensor()
    S.sum(X)
    assert abs(S.s() - total) <= 1e-5 * total, (S.s(), total)
    assert abs(X.sum() - total) <= 1e-5 * total
    assert np.array_equal(X.narrow(1, 17 * chunk + 1, chunk).float(), probe)
