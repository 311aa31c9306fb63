"""Seeded differential runs over randomly laid-out views: every case draws shapes, permuted and
gapped strides and storage offsets, performs the same operation through the THCl API on the GPU
and through the CPU oracle, and compares the WHOLE storages (stray writes are caught too).

The reference's engine accepts any strided operand (src/lib/THClApply.cpp:152-237 pairs elements
by linear index in each tensor's own shape; src/lib/THClReduce.cpp:93-160 reduces any layout);
its own tests only use a handful of hand-written layouts (src/test/unit_tensor.lua), so these
cases widen the coverage of the same contract.

Tolerance: bit-exact for + - * copies, fills and max/min with their indices; 1e-5 relative (of
the sum of magnitudes) for sums, <= 1 ulp or 1e-12 of the running magnitude for scans, 1e-5 in the
Frobenius norm for matrix products.
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.util import Pair

pytestmark = pytest.mark.gpu


def _factor_shape(g, n: int, nd: int):
    """A random shape of `nd` dims whose product is n (n's prime factors dealt out at random)."""
    shape = [1] * nd
    m, p = n, 2
    while m > 1:
        while m % p == 0:
            shape[int(g.integers(nd))] *= p
            m //= p
        p += 1
    return shape


def _random_layout(g, shape, allow_unit_gap=True):
    """(storage length, offset, strides): the dims in a random memory order, each with a random
    gap (so rows are padded / elements are strided), at a random storage offset."""
    nd = len(shape)
    order = list(g.permutation(nd))          # order[0] is the fastest-varying dim in memory
    strides = [0] * nd
    step = int(g.choice([1, 1, 1, 2, 3])) if allow_unit_gap else 1
    for d in order:
        strides[d] = step
        pad = int(g.choice([0, 0, 1, 3, 4]))
        step = step * (shape[d] + pad)
    offset = int(g.choice([0, 0, 1, 3, 4, 16]))
    length = offset + sum((s - 1) * st for s, st in zip(shape, strides)) + 1 + int(g.integers(0, 5))
    return length, offset, strides


def _pair(g, n: int, lo=-1.0, hi=1.0, nd=None, contiguous=False, eighths=False) -> Pair:
    nd = int(g.integers(1, 5)) if nd is None else nd
    shape = _factor_shape(g, n, nd)
    if contiguous:
        length, offset, strides = n, 0, None
    else:
        length, offset, strides = _random_layout(g, shape)
    base = (g.random(length, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)
    if eighths:  # few distinct values: ties
        base = (np.round(base * 8) / 8).astype(np.float32)
    return Pair(base, offset, shape, strides)


# element counts with many factorisations; the larger ones reach the vector, tile and TMA kernels
COUNTS = [1, 2, 7, 24, 210, 840, 4096, 30030, 65536, 2 * 3 * 5 * 7 * 64, 1 << 20, 3 * (1 << 18)]


@pytest.mark.parametrize("seed", range(36))
def test_apply_on_random_views(seed):
    g = np.random.Generator(np.random.PCG64(1000 + seed))
    n = COUNTS[seed % len(COUNTS)]
    r, a, b = _pair(g, n), _pair(g, n), _pair(g, n, 0.5, 2.0)
    tag = f"seed {seed} n {n}: r {r.view.sizes}/{r.view.strides}+{r.view.offset} a {a.view.sizes}/{a.view.strides}+{a.view.offset} " \
          f"b {b.view.sizes}/{b.view.strides}+{b.view.offset}"
    r.cl.add(a.cl); O.apply("ADD_2", [r.view, a.view])
    r.check(0, "add " + tag)
    r.cl.cmul(b.cl); O.apply("MUL_2", [r.view, b.view])
    r.check(0, "cmul " + tag)
    r.cl.addcmul(0.25, a.cl, b.cl); O.apply("ADDCMUL_3", [r.view, a.view, b.view], 0.25)
    r.check(0, "addcmul " + tag)
    r.cl.cdiv(b.cl); O.apply("DIV_2", [r.view, b.view])
    r.check(0, "cdiv " + tag)
    r.cl.copy(a.cl); O.apply("COPY_2", [r.view, a.view])
    r.check(0, "copy " + tag)
    r.cl.mul(1.5); O.apply("MULC_1", [r.view], 1.5)
    r.cl.clamp(-0.75, 0.5); O.apply("CLAMP_1", [r.view], -0.75, 0.5)
    r.check(0, "mul, clamp " + tag)
    a.check(0, "source a untouched " + tag)
    b.check(0, "source b untouched " + tag)


@pytest.mark.parametrize("seed", range(12))
def test_expressions_on_random_views(seed):
    g = np.random.Generator(np.random.PCG64(2000 + seed))
    n = COUNTS[(seed * 5 + 3) % len(COUNTS)]
    r, a, b = _pair(g, n, 0.0, 1.0), _pair(g, n, 0.0, 1.0), _pair(g, n, 0.5, 2.0)
    expr = "x = sqrt(1000 * x + y * 10 + z * z)"                            # + * sqrt only: exactly rounded on both sides
    want = O.eval_expr(expr, r.view.numpy().reshape(-1).copy(), a.view.numpy().reshape(-1).copy(),
                       b.view.numpy().reshape(-1).copy())
    r.cl.map2_on_gpu(a.cl, b.cl, expr)
    r.view.numpy()[...] = np.asarray(want, np.float32).reshape(r.view.sizes)
    r.check(0, f"map2 seed {seed} n {n} {r.view.sizes}/{r.view.strides}")
    a.check(0, "source untouched")


@pytest.mark.parametrize("seed", range(24))
def test_reductions_on_random_views(seed):
    g = np.random.Generator(np.random.PCG64(3000 + seed))
    n = [24, 840, 30030, 65536, 2 * 3 * 5 * 7 * 64, 1 << 20][seed % 6]
    nd = int(g.integers(2, 5))
    a = _pair(g, n, nd=nd, eighths=True)   # values with ties, so that "first occurrence" is exercised
    arr = np.ascontiguousarray(a.view.numpy())
    tag = f"seed {seed} {a.view.sizes}/{a.view.strides}+{a.view.offset}"
    total = a.cl.sum()
    assert abs(total - float(arr.astype(np.float64).sum())) <= 1e-5 * float(np.abs(arr).astype(np.float64).sum()) + 1e-30, tag
    assert a.cl.max() == float(arr.max()) and a.cl.min() == float(arr.min()), tag
    for dim in range(nd):
        got = a.cl.sum(dim + 1).float()
        want = arr.astype(np.float64).sum(axis=dim, keepdims=True)
        scale = np.abs(arr).astype(np.float64).sum(axis=dim, keepdims=True)
        assert got.shape == want.shape, tag
        assert np.all(np.abs(got - want) <= 1e-5 * scale + 1e-30), f"sum({dim + 1}) {tag}"
        for is_max in (True, False):
            v, i = (a.cl.max(dim + 1) if is_max else a.cl.min(dim + 1))
            wv, wi = O.reduce_dim_index(arr, dim, is_max)
            assert np.array_equal(v.float(), wv), f"{'max' if is_max else 'min'}({dim + 1}) values {tag}"
            assert np.array_equal(i.float(), wi), f"{'max' if is_max else 'min'}({dim + 1}) indices {tag}"
    a.check(0, "source untouched " + tag)


@pytest.mark.parametrize("seed", range(12))
def test_scans_on_random_views(seed):
    g = np.random.Generator(np.random.PCG64(4000 + seed))
    n = [840, 30030, 65536, 2 * 3 * 5 * 7 * 64, 1 << 20, 1 << 21][seed % 6]
    nd = int(g.integers(1, 4))
    a = _pair(g, n, -0.5, 0.5, nd=nd, contiguous=seed % 2 == 0)
    arr = np.ascontiguousarray(a.view.numpy())
    for dim in range(nd):
        got = a.cl.cumsum(dim + 1).float()
        want = O.scan(arr, dim, False)
        d = O.ulp_diff(got, want)
        scale = np.cumsum(np.abs(arr.astype(np.float64)), axis=dim)
        bad = (d > 1) & (np.abs(got.astype(np.float64) - want.astype(np.float64)) > 1e-12 * scale)
        assert not bad.any(), f"cumsum({dim + 1}) seed {seed} {a.view.sizes}/{a.view.strides}: {int(bad.sum())} elements off"
    a.check(0, "source untouched")


def _matrix(g, rows: int, cols: int, lo=-1.0, hi=1.0):
    """(ClTensor view, numpy array of its values): row-major, column-major (a transposed view) or a
    window of a wider matrix, at random."""
    import cltorch_b200 as cl
    kind = int(g.integers(3))
    vals = (g.random((rows, cols), dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)
    if kind == 0:
        return cl.ClTensor(vals), vals
    if kind == 1:
        return cl.ClTensor(np.ascontiguousarray(vals.T)).t(), vals
    pad = int(g.choice([1, 3, 4, 8]))
    wide = np.zeros((rows, cols + pad), np.float32)
    wide[:, :cols] = vals
    return cl.ClTensor(wide).narrow(2, 1, cols), vals


@pytest.mark.parametrize("seed", range(30))
def test_addmm_on_random_shapes_and_layouts(seed):
    """THClTensor_addmm (src/lib/THClTensorMathBlas.cpp:107-214) normalises any combination of
    row-major, transposed and padded operands; beta = 0 must not read the result. The contract is 1e-4
    relative; the three-term TF32 split with fp32 accumulation in tensor memory lands at 1e-6 for short K and
    4e-6 to 7e-6 for K in the thousands, so the bar here is 1e-5 in the Frobenius norm and 2e-5 of
    |alpha| |A| |B| + |beta| |C| per element."""
    import cltorch_b200 as cl
    g = np.random.Generator(np.random.PCG64(5000 + seed))
    pick = lambda: int(g.choice([1, 3, 17, 64, 100, 128, 129, 200, 256, 300, 512, 700]))
    M, N = pick(), pick()
    K = int(g.choice([1, 5, 32, 64, 100, 128, 260, 1024, 1100, 2048, 4100]))
    alpha = float(g.choice([1.0, 2.0, -0.5]))
    beta = float(g.choice([0.0, 1.0, 0.5]))
    A, a = _matrix(g, M, K)
    B, b = _matrix(g, K, N)
    R, t = _matrix(g, M, N)
    R.addmm(beta, R, alpha, A, B)
    want = O.addmm(beta, t, alpha, a, b)
    got = R.float()
    tag = f"seed {seed}: {M}x{N}x{K} alpha {alpha} beta {beta} strides A {A.stride()} B {B.stride()} C {R.stride()}"
    err = np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30)
    assert err <= 1e-5, f"{tag}: relative error {err:.3e}"
    scale = abs(alpha) * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)) + abs(beta) * np.abs(t) + 1e-30
    worst = float((np.abs(got.astype(np.float64) - want) / scale).max())
    assert worst <= 2e-5, f"{tag}: worst element error {worst:.3e} of its scale"


@pytest.mark.parametrize("seed", range(18))
def test_moments_norms_renorm_on_random_views(seed):
    """var/std (both normalisations), norm and renorm along every dim of a randomly laid-out view, and
    dist / varall / stdall / normall of it (src/lib/THClTensorMath2.cl:5-143, THClTensorMath2.cpp:293-474)."""
    g = np.random.Generator(np.random.PCG64(6000 + seed))
    n = [840, 30030, 65536, 2 * 3 * 5 * 7 * 64, 1 << 18, 1 << 20][seed % 6]
    nd = int(g.integers(2, 4))
    a = _pair(g, n, -1.0, 1.0, nd=nd)
    b = _pair(g, n, -1.0, 1.0, nd=nd)
    arr = np.ascontiguousarray(a.view.numpy())
    tag = f"seed {seed} {a.view.sizes}/{a.view.strides}+{a.view.offset}"
    a64 = arr.astype(np.float64)
    for dim in range(nd):
        if arr.shape[dim] > 1:
            for flag in (False, True):
                got = a.cl.var(dim + 1, flag).float()
                want = O.var_dim(arr, dim, flag, False)
                assert np.all(np.abs(got - want) <= 2e-5 * np.abs(want) + 1e-7), f"var({dim + 1}, {flag}) {tag}"
                got = a.cl.std(dim + 1, flag).float()
                want = O.var_dim(arr, dim, flag, True)
                assert np.all(np.abs(got - want) <= 2e-5 * np.abs(want) + 1e-7), f"std({dim + 1}, {flag}) {tag}"
        for p in (1.0, 2.0, 3.0):
            got = a.cl.norm(p, dim + 1).float()
            want = (np.abs(a64) ** p).sum(axis=dim, keepdims=True) ** (1.0 / p)
            assert np.all(np.abs(got - want) <= 1e-5 * want + 1e-30), f"norm({p}, {dim + 1}) {tag}"
        norms = (np.abs(np.swapaxes(a64, dim, 0).reshape(arr.shape[dim], -1)) ** 2).sum(axis=1) ** 0.5
        maxnorm = float(np.median(norms))
        if np.abs(norms - maxnorm).min() < 1e-4 * maxnorm:
            maxnorm *= 1.0 + 1e-3                                           # keep every norm clear of the threshold
        got = a.cl.renorm(2.0, dim + 1, maxnorm).float()
        want = O.renorm(arr, 2.0, dim, maxnorm)
        assert np.all(np.abs(got - want) <= 2e-6 * np.abs(want) + 1e-30), f"renorm(2, {dim + 1}) {tag}"
    barr = np.ascontiguousarray(b.view.numpy())
    for p in (1.0, 2.0, 2.5):
        want = O.dist(arr.reshape(-1), barr.reshape(-1), p)
        assert abs(a.cl.dist(b.cl, p) - want) <= 1e-5 * want, f"dist({p}) {tag}"
        want = float((np.abs(a64) ** p).sum() ** (1.0 / p))
        assert abs(a.cl.norm(p) - want) <= 1e-5 * want, f"normall({p}) {tag}"
    var = float(a64.var(ddof=1))
    assert abs(a.cl.var() - var) <= 1e-5 * var and abs(a.cl.std() - var ** 0.5) <= 1e-5 * var ** 0.5, tag
    a.check(0, "source untouched " + tag)
    b.check(0, "source untouched " + tag)


@pytest.mark.parametrize("seed", range(16))
def test_addmv_addr_dot_on_random_layouts(seed):
    """THClTensor_addmv / addr / dot (src/lib/THClTensorMathBlas.cpp:17-105, 216-277) on row-major, transposed
    and padded matrices and strided vectors. Products rounded to fp32, sums in double: 1e-5 of |A||x| + |y|;
    addr rounds like the pointwise operator: bit-exact."""
    import cltorch_b200 as cl
    g = np.random.Generator(np.random.PCG64(7000 + seed))
    M = int(g.choice([1, 3, 100, 129, 512, 2000, 4099]))
    K = int(g.choice([1, 5, 128, 257, 1024, 3000, 8200]))
    A, a = _matrix(g, M, K)

    def vector(length):
        step = int(g.choice([1, 1, 2, 3]))
        base = (g.random(length * step + 2, dtype=np.float32) * 2 - 1).astype(np.float32)
        t = cl.ClTensor(cl.ClStorage(base), 2, [length], [step])
        return t, base[1:1 + length * step:step].copy()

    X, x = vector(K)
    Y, y = vector(M)
    tag = f"seed {seed}: {M}x{K} A strides {A.stride()} x stride {X.stride()} y stride {Y.stride()}"
    beta, alpha = float(g.choice([0.0, 1.0, 0.5])), float(g.choice([1.0, -2.0]))
    R = cl.ClTensor(M)
    R.addmv(beta, Y, alpha, A, X)
    want = beta * y.astype(np.float64) + alpha * (a.astype(np.float64) @ x.astype(np.float64))
    scale = abs(alpha) * (np.abs(a).astype(np.float64) @ np.abs(x).astype(np.float64)) + abs(beta) * np.abs(y) + 1e-30
    assert np.all(np.abs(R.float() - want) <= 1e-5 * scale), "addmv " + tag
    At = A.t()
    R2 = cl.ClTensor(K)
    R2.addmv(0.0, X, 1.0, At, Y)
    want = a.astype(np.float64).T @ y.astype(np.float64)
    scale = np.abs(a).astype(np.float64).T @ np.abs(y).astype(np.float64) + 1e-30
    assert np.all(np.abs(R2.float() - want) <= 1e-5 * scale), "addmv of the transposed view " + tag
    want = float(x.astype(np.float64) @ x.astype(np.float64))
    assert abs(X.dot(X) - want) <= 1e-6 * want + 1e-30, "dot " + tag
    Rm, rm = _matrix(g, M, K)
    Rm.addr(0.5, Rm, 2.0, Y, X)
    want = (np.float32(0.5) * rm + np.float32(2.0) * (y[:, None] * x[None, :]).astype(np.float32)).astype(np.float32)
    got = Rm.float()
    assert O.ulp_diff(got, want).max() <= 1, "addr " + tag
