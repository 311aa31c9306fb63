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
                                   (512, 1024, 256), (1000, 130, 1000)])
def test_addmm_shapes(M, N, K):
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


def test_gemm_status_word_reports_completion():
    import ctypes as C
    import cltorch_b200 as cl
    a = cl.ClTensor(rng_uniform(41, (64, 64)))
    r = cl.ClTensor().mm(a, a)
    cl.synchronize()
    assert np.isfinite(r.float()).all()
