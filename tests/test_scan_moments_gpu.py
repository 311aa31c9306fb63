"""Parity of var/std along a dimension, varall/stdall, cumsum/cumprod, renorm and dist
against the CPU oracle, through the THCl C API and (for argument checks) the thin C ABI.

Tolerances: variances, norms and distances within 1e-5 relative of a double-precision
evaluation; scans within 1 fp32 ulp of the double-precision running value (both sides keep
the running value in double; only the grouping of the additions differs).
"""

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import rng_uniform

pytestmark = pytest.mark.gpu


def normal(seed, shape, mean=0.0, std=1.0):
    g = np.random.Generator(np.random.PCG64(seed))
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).astype(np.float32)


def assert_rel(got, want, tol=1e-5, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = np.abs(got - want) / np.maximum(np.abs(want), 1e-30)
    assert err.max() <= tol, f"{what}: max relative error {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}"


# ---- var / std -------------------------------------------------------------------------------

VAR_SHAPES = [((50, 60), 0), ((50, 60), 1), ((7, 33, 20), 0), ((7, 33, 20), 1), ((7, 33, 20), 2), ((1000, 4096), 0),
              ((1000, 4096), 1), ((20000, 12), 0), ((3, 100001), 1), ((300, 1003), 0), ((5, 8192 + 4), 1),
              # enough 128-column strips for the TMA pipeline (chunked rows, ragged strip, outer > 1)
              ((4096, 2048), 0), ((3000, 5000), 0), ((64, 512, 1024), 1)]


@pytest.mark.parametrize("shape,dim", VAR_SHAPES)
@pytest.mark.parametrize("flag", [False, True])
def test_var_std_dim(shape, dim, flag):
    import cltorch_b200 as cl
    a = normal(31, shape, mean=3.0, std=2.0)
    t = cl.ClTensor(a)
    v = t.var(dim + 1, flag)
    s = t.std(dim + 1, flag)
    want_shape = list(shape)
    want_shape[dim] = 1
    assert list(v.size()) == want_shape and list(s.size()) == want_shape      # the dimension stays, with size 1
    assert_rel(v.float(), O.var_dim(a, dim, flag, False), what="var")
    assert_rel(s.float(), O.var_dim(a, dim, flag, True), what="std")


def test_var_dim_far_from_zero_mean():
    """mean / std = 1e5: the sums are taken about the first element of each slice, so nothing cancels."""
    import cltorch_b200 as cl
    a = normal(32, (4096, 300), mean=1.0e5, std=1.0)
    for dim in (0, 1):
        assert_rel(cl.ClTensor(a).var(dim + 1).float(), O.var_dim(a, dim), tol=1e-5, what=f"dim {dim}")
    t = cl.ClTensor(a)
    assert_rel([t.var()], O.var_dim(a.reshape(1, -1), 1).reshape(1), what="varall")
    assert_rel([t.std()], O.var_dim(a.reshape(1, -1), 1, False, True).reshape(1), what="stdall")


def test_var_dim_strided_source_and_result_argument():
    import cltorch_b200 as cl
    a = normal(33, (60, 50))
    t = cl.ClTensor(a)
    r = cl.ClTensor()
    r.var(t.t(), 1)                                            # result-first form over a transposed view
    assert_rel(r.float(), O.var_dim(a.T, 0), what="transposed")
    w = t.narrow(2, 5, 20)
    assert_rel(w.std(2, True).float(), O.var_dim(a[:, 4:24], 1, True, True), what="narrowed")
    # constant slices: variance exactly 0 (clamped), also for n = 1 with flag (divide by n)
    c = cl.ClTensor(np.full((6, 9), 2.5, np.float32))
    assert np.array_equal(c.var(1).float(), np.zeros((1, 9), np.float32))
    assert np.array_equal(cl.ClTensor(np.ones((1, 4), np.float32)).var(1, True).float(), np.zeros((1, 4), np.float32))


def test_varall_point_tensor_form_matches_host_form():
    import cltorch_b200 as cl
    a = normal(34, (1 << 20) + 3, mean=-2.0, std=0.5)
    t = cl.ClTensor(a)
    pv, ps = cl.ClTensor(), cl.ClTensor()
    pv.var(t)
    ps.std(t)
    assert pv.s() == t.var() and ps.s() == t.std()
    assert_rel([t.var()], [a.astype(np.float64).var(ddof=1)], what="varall")


# ---- cumsum / cumprod ------------------------------------------------------------------------

SCAN_SHAPES = [((50, 60), 0), ((50, 60), 1), ((3, 1000, 7), 1), ((3, 1000, 8), 1), ((4, 100000), 1), ((4, 100003), 1),
               ((100000, 8), 0), ((100000, 3), 0), ((1 << 22,), 0), (((1 << 22) + 5,), 0), ((2000, 129), 1),
               ((2000, 128), 1), ((1, 1), 0), ((5, 1), 1), ((1, 9), 0), ((33000, 40), 0),
               # few thousand columns and many rows: one pass over 128-column strips (ragged last strip, ragged rows)
               ((2000, 12800), 0), ((1000, 12700), 0), ((12, 500, 1028), 1), ((70, 16384), 0),
               # few long rows: single pass over 8192-element tiles that wait for their carries (rows that end
               # inside a round of tiles, ragged last tiles, fewer tiles than SMs, more than one round)
               ((3, (1 << 20) + 32), 1), ((3, (1 << 20) + 4), 1), ((1 << 24,), 0), ((7, 81920), 1), ((2, 16384), 1), ((150, 40000), 1),
               # one vector of any length: the elements after the last multiple of 32 follow in a second kernel
               (((1 << 20) + 17,), 0), ((1, 16384 + 31), 1)]


def scan_close(got, want_f32, src, dim, is_mul, what):
    got = np.asarray(got, np.float32)
    assert got.shape == want_f32.shape, (what, got.shape, want_f32.shape)
    d = O.ulp_diff(got, want_f32)
    if d.size == 0 or d.max() <= 1:
        return
    assert not is_mul, f"{what}: max ulp distance {int(d.max())}"
    # where a running sum nearly cancels it is tiny against the terms added so far: allow the
    # difference between two groupings of the same double-precision additions
    scale = np.cumsum(np.abs(src.astype(np.float64)), axis=dim)
    bad = (d > 1) & (np.abs(got.astype(np.float64) - want_f32.astype(np.float64)) > 1e-12 * scale)
    assert not bad.any(), f"{what}: {int(bad.sum())} elements differ by more than 1 ulp (max {int(d.max())})"


@pytest.mark.parametrize("shape,dim", SCAN_SHAPES)
def test_cumsum_cumprod(shape, dim):
    import cltorch_b200 as cl
    a = rng_uniform(41, shape, -0.5, 0.5)
    got = cl.ClTensor(a).cumsum(dim + 1)
    assert list(got.size()) == list(shape)
    scan_close(got.float(), O.scan(a, dim, False), a, dim, False, "cumsum")
    # products of numbers near 1, so that long prefixes neither overflow nor vanish
    b = rng_uniform(42, shape, 0.999, 1.001)
    scan_close(cl.ClTensor(b).cumprod(dim + 1).float(), O.scan(b, dim, True), b, dim, True, "cumprod")


def test_scan_in_place_default_dim_and_strided_operands():
    import cltorch_b200 as cl
    a = rng_uniform(43, (70, 90), -0.5, 0.5)
    t = cl.ClTensor(a)
    assert np.array_equal(t.cumsum().float(), t.cumsum(1).float())          # default: first dimension
    r = cl.ClTensor(a)
    r.cumsum(r, 2)                                                           # result is the source
    scan_close(r.float(), O.scan(a, 1, False), a, 1, False, "in place")
    tt = t.t()                                                               # non-contiguous source
    scan_close(tt.cumsum(1).float(), O.scan(np.ascontiguousarray(a.T), 0, False), a.T, 0, False, "transposed source")
    out = cl.ClTensor(90, 70).t()                                            # non-contiguous result, same shape as src
    out.cumprod(t, 2)
    assert list(out.size()) == [70, 90]
    scan_close(out.float(), O.scan(a, 1, True), a, 1, True, "transposed result")


def test_strip_scan_in_place_and_status_word():
    import cltorch_b200 as cl
    a = rng_uniform(48, (700, 12804), -0.5, 0.5)
    r = cl.ClTensor(a)
    r.cumsum(r, 1)                                                           # in place along the rows: the strip path
    scan_close(r.float(), O.scan(a, 0, False), a, 0, False, "strips, in place")
    cl.synchronize()                                                         # reads the kernels' status word: must be 0


def test_chained_scan_in_place_repeatable_and_status_word():
    import cltorch_b200 as cl
    a = rng_uniform(49, (2, (1 << 21) + 96), -0.5, 0.5)
    want = O.scan(a, 1, False)
    r = cl.ClTensor(a)
    r.cumsum(r, 2)                                                           # in place: a tile is loaded before it is stored
    first = r.float()
    scan_close(first, want, a, 1, False, "chained, in place")
    for _ in range(3):                                                       # the order of the additions is fixed
        assert np.array_equal(cl.ClTensor(a).cumsum(2).float(), first)
    cl.synchronize()                                                         # reads the kernels' status word: must be 0


def test_scan_abi_rejects_bad_arguments():
    import cltorch_b200 as cl
    from cltorch_b200 import _lib
    L = _lib.load()
    x = cl.ClTensor(rng_uniform(44, (4, 100000)))
    ptr = x.data_ptr()
    need = L.thb200_scan_scratch_bytes(ptr, ptr, 4, 100000, 1)
    assert need > 0                                                          # 4 rows: the rows are cut into chunks
    assert L.thb200_scan(None, 0, ptr, ptr, 4, 100000, 1, None, 0, None) != 0
    assert b"scratch" in L.thb200_last_error()
    assert L.thb200_scan(None, 3, ptr, ptr, 4, 100000, 1, None, 0, None) != 0      # RED_MAX is not a scan operator
    assert b"neither add nor mul" in L.thb200_last_error()
    assert L.thb200_scan(None, 0, ptr, ptr, 0, 100000, 1, None, 0, None) == 0      # empty: nothing to do


# ---- renorm ----------------------------------------------------------------------------------

# rows of 300 (a warp per row), 200, 40 * 20 = 800, 8200 (a CTA per row), 20000 (two kernels), 301 (not a multiple of 4:
# two kernels), 8 / 24 / 32 (8, 8 and 16 lanes per row), 100, 2048 (16 vectors per lane)
@pytest.mark.parametrize("shape,dim", [((200, 300), 0), ((200, 300), 1), ((20, 30, 40), 1), ((64, 8192 + 8), 0),
                                       ((40, 20000), 0), ((50, 301), 0), ((3000, 64), 0), ((300, 1500), 0), ((90, 4000), 0),
                                       ((5000, 8), 0), ((777, 24), 0), ((1001, 32), 0), ((333, 100), 0), ((67, 2048), 0)])
@pytest.mark.parametrize("p", [1.0, 2.0, 3.0])
def test_renorm(shape, dim, p):
    import cltorch_b200 as cl
    a = normal(51, shape)
    moved = np.ascontiguousarray(np.swapaxes(a, dim, 0)).reshape(shape[dim], -1).astype(np.float64)
    norms = (np.abs(moved) ** p).sum(axis=1) ** (1.0 / p)
    maxnorm = float(np.median(norms))
    gap = np.abs(norms - maxnorm) / maxnorm
    maxnorm *= 1.0 + 1e-3 if gap.min() < 1e-4 else 1.0                      # keep every norm clear of the threshold
    want = O.renorm(a, p, dim, maxnorm)
    assert 0 < (want != a).any(axis=tuple(k for k in range(a.ndim) if k != dim)).sum() < shape[dim]   # some rows scaled, some not
    t = cl.ClTensor(a)
    out = t.renorm(p, dim + 1, maxnorm)
    assert list(out.size()) == list(shape)
    assert_rel(out.float(), want, tol=2e-6, what="out of place")
    assert np.array_equal(t.float(), a)                                      # the source is untouched
    t.renorm(t, p, dim + 1, maxnorm)                                         # in place
    assert_rel(t.float(), want, tol=2e-6, what="in place")
    untouched = want == a
    assert np.array_equal(t.float()[untouched], a[untouched])                # rows within the limit are bit-identical


@pytest.mark.parametrize("shape", [(100, 256), (30, 5000), (12, 30000)])
def test_renorm_general_power_and_zero_limit(shape):
    import cltorch_b200 as cl
    a = normal(54, shape)
    norms = (np.abs(a.astype(np.float64)) ** 2.5).sum(axis=1) ** (1.0 / 2.5)
    maxnorm = float(np.median(norms)) * (1.0 + 1e-3)
    out = cl.ClTensor(a).renorm(2.5, 1, maxnorm)
    assert_rel(out.float(), O.renorm(a, 2.5, 0, maxnorm), tol=1e-5, what="p = 2.5 (power on the special-function unit)")
    # a limit of zero scales every row with a positive norm to zero; an all-zero row has norm 0, not above the limit
    b = a.copy()
    b[3] = 0.0
    z = cl.ClTensor(b).renorm(2.0, 1, 0.0).float()
    assert np.array_equal(z, np.zeros_like(b) * b)                           # signed zeros as x * 0 gives them
    assert np.array_equal(z[3], b[3])


def test_renorm_argument_checks():
    import cltorch_b200 as cl
    t = cl.ClTensor(normal(52, (4, 5)))
    with pytest.raises(cl.ClError, match="invalid dimension"):
        t.renorm(2, 3, 1.0)
    with pytest.raises(cl.ClError, match="non-positive-norm"):
        t.renorm(0, 1, 1.0)
    with pytest.raises(cl.ClError, match="at least 2 dimensions"):
        cl.ClTensor(normal(53, (7,))).renorm(2, 1, 1.0)


# ---- dist ------------------------------------------------------------------------------------

@pytest.mark.parametrize("n", [1, 5, 1000, (1 << 20) + 3])
@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, 4.0, 0.5])
def test_dist(n, p):
    import cltorch_b200 as cl
    a, b = normal(61, (n,)), normal(62, (n,))
    ta, tb = cl.ClTensor(a), cl.ClTensor(b)
    assert_rel([ta.dist(tb, p)], [O.dist(a, b, p)], what="dist")
    pt = cl.ClTensor().dist_gpu(ta, tb, p)
    assert pt.s() == ta.dist(tb, p)
    if n > 8:                                                                # unaligned, strided operands
        va, vb = ta.narrow(1, 2, n - 3), tb.narrow(1, 3, n - 3)
        assert_rel([va.dist(vb, p)], [O.dist(a[1:n - 2], b[2:n - 1], p)], what="dist of narrowed views")


def test_dist_default_is_euclidean_and_sizes_must_match():
    import cltorch_b200 as cl
    a, b = normal(63, (30, 40)), normal(64, (30, 40))
    ta, tb = cl.ClTensor(a), cl.ClTensor(b)
    assert_rel([ta.dist(tb)], [np.sqrt(((a.astype(np.float64) - b) ** 2).sum())], what="p = 2")
    assert_rel([ta.t().dist(tb.t(), 1)], [np.abs(a.astype(np.float64) - b).sum()], tol=1e-5, what="transposed views")
    with pytest.raises(cl.ClError, match="sizes do not match"):
        ta.dist(cl.ClTensor(normal(65, (30, 41))))
