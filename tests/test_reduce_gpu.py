"""Parity of reduceAll (host scalars and point tensors), reduceDim and max/min with
indices against the CPU oracle, through the THCl C API.

Tolerances: sums, means, products and norms within 1e-5 relative of a double-precision
evaluation; max/min values and every index bit-exact (ties: first occurrence).
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.util import Pair, rng_uniform

pytestmark = pytest.mark.gpu

M23 = np.array([[3, 2, 4], [9, 7, 5]], dtype=np.float32)   # unit_tensor.lua:488-496


def rel(a, b):
    return abs(a - b) / max(abs(b), 1e-30)


def test_matrixwide_known_answers():
    import cltorch_b200 as cl
    c = cl.ClTensor(M23)
    assert c.max() == 9.0 and c.min() == 2.0 and c.sum() == 30.0 and c.prod() == 3 * 2 * 4 * 9 * 7 * 5
    assert np.array_equal(c.sum(1).float(), [[12, 9, 9]])
    assert np.array_equal(c.sum(2).float(), [[9], [21]])
    assert c.mean() == 5.0
    assert c.all() is True and c.any() is True
    z = cl.ClTensor(np.array([[0, 1], [2, 0]], np.float32))
    assert z.all() is False and z.any() is True
    assert cl.ClTensor(np.zeros((2, 2), np.float32)).any() is False
    assert z.norm(0) == 2.0 and rel(z.norm(2), np.sqrt(5.0)) < 1e-6 and rel(z.norm(1), 3.0) < 1e-6


@pytest.mark.parametrize("n", [1, 2, 31, 32, 33, 1000, 2000, 4097, 50 * 40, 28 * 28 * 1280 * 10])
def test_sumall_one_and_two_pass(n):
    import cltorch_b200 as cl
    a = rng_uniform(21, (n,), -0.5, 0.5)                   # unit_tensor.lua:637-657
    want = O.reduce_all(O.View(a))
    got = cl.ClTensor(a).sum()
    assert abs(got - want) <= 1e-5 * max(abs(want), np.abs(a.astype(np.float64)).sum() * 1e-2, 1e-6), (got, want)
    b = rng_uniform(22, (n,), 0.5, 1.5)
    assert rel(cl.ClTensor(b).sum(), O.reduce_all(O.View(b))) < 1e-5
    assert cl.ClTensor(b).max() == b.max() and cl.ClTensor(b).min() == b.min()


def test_reduce_all_strided_and_offset():
    import cltorch_b200 as cl
    base = rng_uniform(23, (60, 50), 0.5, 1.5)
    a = cl.ClTensor(base)
    for view, ref in [(a.t(), base.T), (a.narrow(1, 10, 30).t(), base[9:39].T), (a.narrow(2, 10, 30), base[:, 9:39]),
                      (a.narrow(2, 4, 1), base[:, 3:4])]:
        want = float(ref.astype(np.float64).sum())
        assert rel(view.sum(), want) < 1e-5
        assert view.max() == ref.max() and view.min() == ref.min()
    p = rng_uniform(24, (7, 5), 0.9, 1.1)
    assert rel(cl.ClTensor(p).prod(), float(np.prod(p.astype(np.float64)))) < 1e-5


def test_point_tensors_stay_on_device():
    import cltorch_b200 as cl
    c = rng_uniform(25, (20, 30))                          # README.md:125-138
    C = cl.ClTensor(c)
    res = cl.ClTensor()
    assert res.dim() == -1
    res.sum(C)
    assert res.dim() == 0 and res.nElement() == 0
    total = O.reduce_all(O.View(c))
    assert rel(res.s(), total) < 1e-5
    s32 = np.float32(res.s())
    C.div(res)                                             # true division by the device-resident scalar
    assert np.array_equal(C.float(), c / s32)
    # scalar div multiplies by the reciprocal instead
    C2 = cl.ClTensor(c).div(float(s32))
    assert np.array_equal(C2.float(), c * (np.float32(1.0) / s32))
    for name, fn in [("prod", np.prod), ("min", np.min), ("max", np.max)]:
        r = cl.ClTensor()
        getattr(r, name)(cl.ClTensor(c[:3, :4] + 0.5))
        assert rel(r.s(), float(fn((c[:3, :4] + np.float32(0.5)).astype(np.float64)))) < 1e-5
    # add / csub / mul / fill / compare with a point tensor (test-tensor.lua:809-934)
    m = cl.ClTensor(); m.max(cl.ClTensor(c))
    mx = c.max()
    assert np.array_equal(cl.ClTensor(c).add(m).float(), c + mx)
    assert np.array_equal(cl.ClTensor(c).csub(m).float(), c - mx)
    assert np.array_equal(cl.ClTensor(c).mul(m).float(), c * mx)
    assert np.array_equal(cl.ClTensor(3, 2).fill(m).float(), np.full((3, 2), mx, np.float32))
    assert np.array_equal(cl.ClTensor(c).ge(m).float(), (c >= mx).astype(np.float32))
    # logical all/any cast to int first ("(int)*in1 && (int)*in2"): 0.5 counts as false
    a_all = cl.ClTensor(); a_all.all(cl.ClTensor(c + 1))
    assert a_all.s() == 1.0
    a_all.all(cl.ClTensor(c))
    assert a_all.s() == 0.0
    a_any = cl.ClTensor(); a_any.any(cl.ClTensor(c))
    assert a_any.s() == 0.0


def test_mean_std_var_point_tensors_and_chain():
    import cltorch_b200 as cl
    a = np.random.Generator(np.random.PCG64(26)).standard_normal((257, 129)).astype(np.float32) * 3 + 2
    A = cl.ClTensor(a)
    a64 = a.astype(np.float64)
    assert rel(A.mean(), a64.mean()) < 1e-5
    assert rel(A.std(), a64.std(ddof=1)) < 1e-5 and rel(A.var(), a64.var(ddof=1)) < 1e-5
    m, s = cl.ClTensor(), cl.ClTensor()
    for _ in range(3):                                     # a:add(-a:mean()):div(a:std()) kept on the device
        m.mean(A); A.csub(m); s.std(A); A.div(s)
    out = A.float().astype(np.float64)
    assert abs(out.mean()) < 1e-5 and rel(out.std(ddof=1), 1.0) < 1e-5


SHAPES = [(60, 50), (5, 2), (1, 7), (7, 1), (3, 1025), (1025, 3), (4, 5, 6), (2, 300, 7), (33, 2, 2, 9), (2100, 130)]
# reductions over a non-innermost dimension with enough 128-column strips for the TMA pipeline:
# several row chunks, a ragged last strip (5000 = 39 * 128 + 8), a ragged last row block, outer > 1
STRIP_SHAPES = [(4096, 2048), (3000, 5000), (64, 512, 1024), (300, 20000), (2, 1000, 9600)]


@pytest.mark.parametrize("shape", SHAPES + STRIP_SHAPES)
def test_sum_prod_mean_each_dim(shape):
    import cltorch_b200 as cl
    a = rng_uniform(27, shape, 0.9, 1.1)
    A = cl.ClTensor(a)
    for d in range(len(shape)):
        want = a.astype(np.float64).sum(axis=d, keepdims=True)
        got = A.sum(d + 1).float()
        assert got.shape == want.shape
        assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want))
        assert np.all(np.abs(A.mean(d + 1).float() - want / shape[d]) <= 2e-5 * np.abs(want / shape[d]))
        if a.shape[d] <= 64:
            wantp = a.astype(np.float64).prod(axis=d, keepdims=True)
            assert np.all(np.abs(A.prod(d + 1).float() - wantp) <= 1e-5 * np.abs(wantp))


def test_sum_of_transposed_and_narrowed_views():
    import cltorch_b200 as cl
    a = rng_uniform(28, (60, 50), -0.5, 0.5)               # unit_tensor.lua:759-775
    A = cl.ClTensor(a)
    cases = [(A.t(), a.T), (A.narrow(1, 10, 30).t(), a[9:39].T), (A.narrow(2, 10, 30).t(), a[:, 9:39].T),
             (A.narrow(2, 10, 30), a[:, 9:39])]
    for view, ref in cases:
        for d in (1, 2):
            want = ref.astype(np.float64).sum(axis=d - 1, keepdims=True)
            got = view.sum(d).float()
            assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1.0))
    # oracle agreement on the same strided view
    ov = O.View.of(a[9:39].T)
    assert np.allclose(O.reduce_dim(ov, 0), a[9:39].T.astype(np.float64).sum(axis=0, keepdims=True), rtol=1e-6)


def test_norm_along_dim():
    import cltorch_b200 as cl
    a = rng_uniform(29, (40, 30), -1, 1)
    A = cl.ClTensor(a)
    for p in (1.0, 2.0, 3.0, 4.0, 2.5, 0.5):
        want = (np.abs(a.astype(np.float64)) ** p).sum(axis=1, keepdims=True) ** (1 / p)
        assert np.all(np.abs(A.norm(p, 2).float() - want) <= 1e-5 * want)
    assert np.array_equal(A.norm(0, 1).float(), (a != 0).sum(axis=0, keepdims=True).astype(np.float32))


@pytest.mark.parametrize("shape", SHAPES + STRIP_SHAPES + [(5, 2, 1), (1, 1), (70000, 3), (3, 70000)])
def test_max_min_with_indices_each_dim(shape):
    import cltorch_b200 as cl
    g = np.random.Generator(np.random.PCG64(30))
    a = g.integers(-5, 6, size=shape).astype(np.float32)   # many exact ties
    A = cl.ClTensor(a)
    for d in range(len(shape)):
        for name, is_max in (("max", True), ("min", False)):
            v, i = getattr(A, name)(d + 1)
            wv, wi = O.reduce_dim_index(a, d, is_max)
            assert np.array_equal(v.float(), wv), (name, d)
            assert np.array_equal(i.float(), wi), (name, d)
            # independent statement of the rule: first occurrence, 1-based
            first = (a.argmax(axis=d) if is_max else a.argmin(axis=d)) + 1
            assert np.array_equal(i.long().squeeze(d), first)


@pytest.mark.parametrize("shape", [(5, 7), (300, 257), (3000, 5000), (4096, 2048), (70000, 3), (3, 70000)])
def test_max_min_of_a_transposed_view_runs_on_the_storage_as_it_lies(shape):
    """max / min of A:t() along either dimension: same values and 1-based positions as for a contiguous copy of the
    transposed matrix (the front-end reduces the matrix underneath along the other dimension instead of copying)."""
    import cltorch_b200 as cl
    g = np.random.Generator(np.random.PCG64(36))
    a = g.integers(-9, 10, size=shape).astype(np.float32)
    a[0, 0] = np.nan
    At = cl.ClTensor(a).t()
    at = np.ascontiguousarray(a.T)
    for d in (0, 1):
        for name, is_max in (("max", True), ("min", False)):
            v, i = getattr(At, name)(d + 1)
            wv, wi = O.reduce_dim_index(at, d, is_max)
            assert tuple(v.size()) == tuple(wv.shape) and v.isContiguous()
            assert np.array_equal(v.float(), wv), (name, d)
            assert np.array_equal(i.float(), wi), (name, d)
    assert np.array_equal(At.float()[1:], at[1:])                        # the source is untouched


def test_max_min_index_corner_cases():
    import cltorch_b200 as cl
    a = np.array([[np.nan, 1, 3, 3], [-np.inf, -np.inf, -np.inf, -np.inf], [2, np.nan, 2, 1]], np.float32)
    A = cl.ClTensor(a)
    v, i = A.max(2)
    wv, wi = O.reduce_dim_index(a, 1, True)
    assert np.array_equal(v.float(), wv) and np.array_equal(i.float(), wi)
    # NaN never replaces the running value; a slice with nothing above -FLT_MAX keeps index -1
    assert list(i.float().ravel()) == [3.0, -1.0, 1.0]
    v, i = A.min(1)
    wv, wi = O.reduce_dim_index(a, 0, False)
    assert np.array_equal(v.float(), wv) and np.array_equal(i.float(), wi)
    # strided source: the front-end makes it contiguous first
    v, i = A.t().max(1)
    wv, wi = O.reduce_dim_index(np.ascontiguousarray(a.T), 0, True)
    assert np.array_equal(v.float(), wv) and np.array_equal(i.float(), wi)


def test_max_min_corner_cases_on_the_strip_path():
    """The same corners on a shape that streams through the TMA strip pipeline in several row chunks."""
    import cltorch_b200 as cl
    g = np.random.Generator(np.random.PCG64(35))
    a = g.integers(-3, 4, size=(3000, 5000)).astype(np.float32)
    a[:, 7] = np.nan                     # a column of NaN only: (-FLT_MAX, -1)
    a[:, 130] = -np.inf                  # nothing above -FLT_MAX: index -1 for max, first row for min
    a[5:, 4999] = np.nan                 # NaN after real values, in the ragged last strip
    a[::2, 640] = np.inf
    a[2999, 1000] = 100.0                # the extreme in the last row of the last chunk
    a[0, 1001] = -100.0                  # ... and in the very first row
    A = cl.ClTensor(a)
    for name, is_max in (("max", True), ("min", False)):
        v, i = getattr(A, name)(1)
        wv, wi = O.reduce_dim_index(a, 0, is_max)
        assert np.array_equal(v.float(), wv) and np.array_equal(i.float(), wi), name
    v, i = A.max(1)
    assert i.float()[0, 7] == -1.0 and i.float()[0, 130] == -1.0 and i.float()[0, 1000] == 3000.0


def test_errors():
    import cltorch_b200 as cl
    A = cl.ClTensor(np.ones((2, 3), np.float32))
    with pytest.raises(cl.ClError, match="out of range"):
        A.sum(3)
    with pytest.raises(cl.ClError, match="out of range"):
        A.max(0)
    with pytest.raises(cl.ClError, match="point tensor"):
        A.s()
