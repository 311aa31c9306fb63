"""addmm / baddbmm / mm / bmm against an fp64-accumulated CPU GEMM, through the THCl C API.

Tolerance: relative error <= 1e-4 in the Frobenius norm and per element relative to the
row/column scale; the three-term TF32 split is expected to land near 1e-6.
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.util import rng_uniform

pytestmark = pytest.mark.gpu


def check(got, want, what, tol=1e-4):
    err = np.linalg.norm(got.astype(np.float64) - want.astype(np.float64)) / max(np.linalg.norm(want.astype(np.float64)), 1e-30)
    assert err <= tol, f"{what}: relative error {err:.3e}"
    scale = np.abs(want.astype(np.float64)).max() + 1e-30
    worst = np.abs(got.astype(np.float64) - want.astype(np.float64)).max() / scale
    assert worst <= tol, f"{what}: worst element error {worst:.3e} of the largest entry"
    return err


def test_blas_fixture_from_reference_tests():
    import cltorch_b200 as cl
    C = cl.ClTensor(np.array([[1, 2, -1], [3, 4, 0]], np.float32))      # unit_tensor.lua:413-425
    D = cl.ClTensor(np.array([[0, 1], [1, 2], [4, 5]], np.float32))
    r = cl.ClTensor().mm(C, D)
    assert np.array_equal(r.float(), np.array([[-2, 0], [4, 11]], np.float32))


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (2, 3, 4), (17, 5, 33), (128, 256, 32), (129, 257, 31), (300, 500, 70),
                                   (512, 1024, 256), (1000, 130, 1000), (300, 500, 4100), (128, 256, 2048)])
def test_addmm_shapes(M, N, K):
    # the last three have few output tiles and a long K: they run split along K (2, 4 and 4 ways)
    import cltorch_b200 as cl
    a = rng_uniform(31, (M, K), -1, 1)
    b = rng_uniform(32, (K, N), -1, 1)
    t = rng_uniform(33, (M, N), -1, 1)
    want = O.addmm(0.5, t, 2.0, a, b)
    r = cl.ClTensor().addmm(0.5, cl.ClTensor(t), 2.0, cl.ClTensor(a), cl.ClTensor(b))
    check(r.float(), want, f"addmm {M}x{N}x{K}")
    # beta = 0 must ignore whatever is in the result (including NaN)
    r = cl.ClTensor(np.full((M, N), np.nan, np.float32))
    r.addmm(0.0, r, 1.0, cl.ClTensor(a), cl.ClTensor(b))
    check(r.float(), O.addmm(0.0, t, 1.0, a, b), "beta = 0")


def test_addmm_operand_layouts():
    """Every transposition / stride case of the front-end's normalisation."""
    import cltorch_b200 as cl
    M, N, K = 70, 50, 90
    a = rng_uniform(34, (M, K), -1, 1)
    b = rng_uniform(35, (K, N), -1, 1)
    t = rng_uniform(36, (M, N), -1, 1)
    want = O.addmm(1.0, t, 1.0, a, b)
    A, B = cl.ClTensor(a), cl.ClTensor(b)
    At, Bt = cl.ClTensor(np.ascontiguousarray(a.T)).t(), cl.ClTensor(np.ascontiguousarray(b.T)).t()
    wide = cl.ClTensor(rng_uniform(37, (M, 2 * K)))
    wide_np = wide.float()
    for la, A_ in (("row", A), ("col", At)):
        for lb, B_ in (("row", B), ("col", Bt)):
            r = cl.ClTensor(t.copy())
            r.addmm(A_, B_)
            check(r.float(), want, f"A {la}-major, B {lb}-major")
            rt = cl.ClTensor(np.ascontiguousarray(t.T)).t()          # column-major result
            rt.addmm(A_, B_)
            check(rt.float(), want, f"column-major result, A {la}, B {lb}")
    # operand with neither stride 1: every other column of a wider matrix
    import cltorch_b200
    s = cltorch_b200.ClTensor(wide.storage(), 1, [M, K], [2 * K, 2])
    r = cl.ClTensor(t.copy()).addmm(s, B)
    check(r.float(), O.addmm(1.0, t, 1.0, np.ascontiguousarray(wide_np[:, ::2]), b), "stride-2 operand")
    with pytest.raises(cl.ClError, match="size mismatch"):
        cl.ClTensor(t.copy()).addmm(A, A)


def test_baddbmm_and_bmm():
    import cltorch_b200 as cl
    Bn, M, N, K = 5, 40, 72, 33
    a = rng_uniform(38, (Bn, M, K), -1, 1)
    b = rng_uniform(39, (Bn, K, N), -1, 1)
    t = rng_uniform(40, (Bn, M, N), -1, 1)
    want = O.addmm(1.0, t, 1.0, a, b)
    r = cl.ClTensor(t.copy()).baddbmm(cl.ClTensor(a), cl.ClTensor(b))
    check(r.float(), want, "baddbmm")
    r = cl.ClTensor().bmm(cl.ClTensor(a), cl.ClTensor(b))
    check(r.float(), O.addmm(0.0, t, 1.0, a, b), "bmm")
    # transposed batches
    at = cl.ClTensor(np.ascontiguousarray(a.transpose(0, 2, 1))).transpose(2, 3)
    r = cl.ClTensor(t.copy()).baddbmm(at, cl.ClTensor(b))
    check(r.float(), want, "baddbmm with a transposed batch operand")
    # few tiles per batch and a long K: the batched split-K path (partials per batch, then the fix-up)
    Bn, M, N, K = 3, 130, 260, 1100
    a = rng_uniform(45, (Bn, M, K), -1, 1)
    b = rng_uniform(46, (Bn, K, N), -1, 1)
    t = rng_uniform(47, (Bn, M, N), -1, 1)
    r = cl.ClTensor(t.copy()).baddbmm(0.5, 2.0, cl.ClTensor(a), cl.ClTensor(b))
    check(r.float(), O.addmm(0.5, t, 2.0, a, b), "baddbmm, split along K")


def test_gemm_status_word_reports_completion():
    import ctypes as C
    import cltorch_b200 as cl
    a = cl.ClTensor(rng_uniform(41, (64, 64)))
    r = cl.ClTensor().mm(a, a)
    cl.synchronize()
    assert np.isfinite(r.float()).all()


def test_dot_addmv_addr_fixtures_from_reference_tests():
    import cltorch_b200 as cl
    c, d = cl.ClTensor(np.array([3, 5, 1], np.float32)), cl.ClTensor(np.array([2, 4, 8], np.float32))
    assert c.dot(d) == 34.0                                             # unit_tensor.lua:437-443
    C = np.array([[3, 1, 7], [3, 2, 4], [8, 5, 3]], np.float32)         # unit_tensor.lua:455-460
    dd, e = np.array([3, 2, 5], np.float32), np.array([3, 1, 2], np.float32)
    r = cl.ClTensor().addr(cl.ClTensor(C), cl.ClTensor(dd), cl.ClTensor(e))
    assert np.array_equal(r.float(), C + np.outer(dd, e))
    r = cl.ClTensor().addr(0.5, cl.ClTensor(C), 2.0, cl.ClTensor(dd), cl.ClTensor(e))
    assert np.array_equal(r.float(), 0.5 * C + 2.0 * np.outer(dd, e))
    assert np.array_equal(cl.ClTensor().ger(cl.ClTensor(dd), cl.ClTensor(e)).float(), np.outer(dd, e))


@pytest.mark.parametrize("M,K", [(1, 1), (5, 3), (300, 70), (70, 9000), (9000, 70), (20000, 33), (129, 1025),
                                 # column-major matrices of these sizes stream through the TMA strip pipeline
                                 (2048, 4096), (5000, 3000), (20000, 260)])
def test_addmv_layouts(M, K):
    import cltorch_b200 as cl
    a = rng_uniform(51, (M, K), -1, 1)
    x = rng_uniform(52, (K,), -1, 1)
    t = rng_uniform(53, (M,), -1, 1)
    want = 0.5 * t.astype(np.float64) + 2.0 * (a.astype(np.float64) @ x.astype(np.float64))
    scale = np.abs(a.astype(np.float64)) @ np.abs(x.astype(np.float64)) + 1.0
    A, X, T = cl.ClTensor(a), cl.ClTensor(x), cl.ClTensor(t)
    At = cl.ClTensor(np.ascontiguousarray(a.T)).t()                      # column-major matrix
    for name, mat in (("row-major", A), ("column-major", At)):
        r = cl.ClTensor().addmv(0.5, T, 2.0, mat, X)
        assert np.all(np.abs(r.float() - want) <= 1e-5 * scale), name
    assert np.all(np.abs(cl.ClTensor().mv(A, X).float() - a.astype(np.float64) @ x.astype(np.float64)) <= 1e-5 * scale)
    # strided vector and a matrix with neither stride 1
    x2 = cl.ClTensor(rng_uniform(54, (K, 2), -1, 1))
    xs = x2.select(2, 1)
    wide = cl.ClTensor(rng_uniform(55, (M, 2 * K), -1, 1))
    ms = cl.ClTensor(wide.storage(), 1, [M, K], [2 * K, 2])
    want2 = wide.float()[:, ::2].astype(np.float64) @ x2.float()[:, 0].astype(np.float64)
    r = cl.ClTensor(M).zero().addmv(0.0, 1.0, ms, xs)
    assert np.all(np.abs(r.float() - want2) <= 1e-5 * (np.abs(wide.float()[:, ::2].astype(np.float64)) @ np.abs(x2.float()[:, 0].astype(np.float64)) + 1))
    with pytest.raises(cl.ClError, match="size mismatch"):
        cl.ClTensor().addmv(T, A, T if K != M else cl.ClTensor(K + 1))


@pytest.mark.parametrize("R,Cc", [(300, 500), (1000, 2048), (4, 4), (333, 12)])
def test_addr_layouts_round_like_the_pointwise_operator(R, Cc):
    """r += alpha * v1 (x) v2 is defined by "*out += val1 * *in1 * *in2" (one rounding per operation,
    alpha * v1 first): the 128-bit rank-1 kernel and the pointwise fallback must agree with it bit for bit."""
    import cltorch_b200 as cl
    t = rng_uniform(58, (R, Cc), -1, 1)
    v1, v2 = rng_uniform(59, (R,), -1, 1), rng_uniform(60, (Cc,), -1, 1)
    alpha = np.float32(1.7)
    want = t + ((alpha * v1)[:, None] * v2[None, :]).astype(np.float32)
    V1, V2 = cl.ClTensor(v1), cl.ClTensor(v2)
    r = cl.ClTensor(t.copy()).addr(float(alpha), V1, V2)                       # row-major result
    assert np.array_equal(r.float(), want)
    rt = cl.ClTensor(np.ascontiguousarray(t.T)).t()                            # column-major (transposed) result
    rt.addr(float(alpha), V1, V2)
    assert np.array_equal(rt.float(), want)
    s2 = cl.ClTensor(np.stack([v2, v2], axis=1)).select(2, 1)                  # strided vector: pointwise fallback
    r = cl.ClTensor(t.copy()).addr(float(alpha), V1, s2)
    assert np.array_equal(r.float(), want)
    if Cc > 8:                                                                 # a window of a wider matrix (pitch > columns)
        wide = cl.ClTensor(np.zeros((R, Cc + 8), np.float32))
        w = wide.narrow(2, 5, Cc - 4)                                          # offset 4 elements: 16-byte aligned
        w.copy(cl.ClTensor(np.ascontiguousarray(t[:, :Cc - 4])))
        w.addr(float(alpha), V1, cl.ClTensor(np.ascontiguousarray(v2[:Cc - 4])))
        assert np.array_equal(w.float(), want[:, :Cc - 4])
        assert np.array_equal(wide.float()[:, :4], np.zeros((R, 4), np.float32))  # nothing written outside the window


def test_dot_large_and_strided():
    import cltorch_b200 as cl
    a, b = rng_uniform(56, (3000, 1001), -1, 1), rng_uniform(57, (3000, 1001), -1, 1)
    want = float(np.sum(a.astype(np.float64) * b.astype(np.float64)))
    scale = float(np.sum(np.abs(a.astype(np.float64) * b.astype(np.float64))))
    assert abs(cl.ClTensor(a).dot(cl.ClTensor(b)) - want) <= 1e-6 * scale
    A, B = cl.ClTensor(a), cl.ClTensor(np.ascontiguousarray(b.T))
    assert abs(A.t().dot(B) - want) <= 1e-6 * scale                    # strided operand: contiguous copy first
    with pytest.raises(cl.ClError, match="sizes do not match"):
        A.dot(cl.ClTensor(5))
