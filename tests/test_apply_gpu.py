"""Parity of the pointwise path (built-in operators, copies, user expressions) with the
CPU oracle, through the THCl C API. Mirrors the structure of the reference's
src/test/unit_tensor.lua: same literal inputs, every operator in and out of place,
plus the strided / offset / overlapping layouts the reference's engine supports.

Tolerance: bit-exact for operators made of + - * / sqrt, compares, copies and fills;
<= 2 ulp for transcendental functions (the bar for pointwise fp32 results).
"""
import itertools

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import Pair, rng_uniform

pytestmark = pytest.mark.gpu

A23 = np.array([[4, 2, -1], [3.1, 1.2, 4.9]], dtype=np.float32)      # unit_tensor.lua:225-228
B23 = np.array([[3, 5, -2], [2.1, 2.2, 3.9]], dtype=np.float32)
C23 = np.array([[4, 2, -1], [0.8, 1.2, 1.9]], dtype=np.float32)      # unit_tensor.lua:267-270
D23 = np.array([[3, 5, -2], [2.1, 2.2, 0.9]], dtype=np.float32)

UNARY = {  # method name -> (operator stem, max ulp)
    "abs": ("ABS", 0), "sqrt": ("SQRT", 0), "log": ("LOG", 2), "exp": ("EXP", 2), "cos": ("COS", 2),
    "acos": ("ACOS", 2), "sin": ("SIN", 2), "asin": ("ASIN", 2), "atan": ("ATAN", 2), "tanh": ("TANH", 2),
    "ceil": ("CEIL", 0), "floor": ("FLOOR", 0), "round": ("ROUND", 0), "sign": ("SIGN", 0), "sigmoid": ("SIGMOID", 2),
    "cinv": ("CINV", 0), "neg": ("NEG", 0), "log1p": ("LOG1P", 2), "cosh": ("COSH", 2), "sinh": ("SINH", 2),
    "tan": ("TAN", 2),
}


@pytest.mark.parametrize("name", sorted(UNARY))
def test_unary_inplace_and_outplace(name):
    stem, ulp = UNARY[name]
    with np.errstate(all="ignore"):
        p = Pair(A23)
        getattr(p.cl, name)()
        O.apply(f"{stem}_1", [p.view])
        p.check(ulp, f"{name} in place")

        src, dst = Pair(A23), Pair(np.zeros_like(A23))
        getattr(dst.cl, name)(src.cl)
        O.apply(f"{stem}_2", [dst.view, src.view])
        dst.check(ulp, f"{name} out of place")
        src.check(0, f"{name}: source untouched")


@pytest.mark.parametrize("name", sorted(UNARY))
def test_unary_wide_range(name):
    """Dense samples over the function's natural domain (4 Mi values)."""
    stem, ulp = UNARY[name]
    g = np.random.Generator(np.random.PCG64(11))
    n = 1 << 22
    if name in ("acos", "asin"):
        x = g.uniform(-1, 1, n)
    elif name in ("log", "sqrt", "cinv"):
        x = np.exp(g.uniform(-20, 20, n))
    elif name in ("exp", "sinh", "cosh", "tanh", "sigmoid"):
        x = g.uniform(-12, 12, n)
    elif name == "log1p":
        x = np.expm1(g.uniform(-10, 10, n))
    else:
        x = g.uniform(-30, 30, n)
    x = x.astype(np.float32)
    with np.errstate(all="ignore"):
        p = Pair(x)
        getattr(p.cl, name)()
        O.apply(f"{stem}_1", [p.view])
        p.check(ulp, f"{name} wide range")


BINARY = [("add", "ADD", 0), ("csub", "SUB", 0), ("cmul", "MUL", 0), ("cdiv", "DIV", 0), ("cpow", "CPOW", 2),
          ("cmax", "CMAX", 0), ("cmin", "CMIN", 0)]


@pytest.mark.parametrize("method,stem,ulp", BINARY)
def test_binary_inplace_and_outplace(method, stem, ulp):
    with np.errstate(all="ignore"):
        c, d = Pair(C23), Pair(D23)
        getattr(c.cl, method)(d.cl)
        O.apply(f"{stem}_2", [c.view, d.view])
        c.check(ulp, f"{method} in place")

        c, d, r = Pair(C23), Pair(D23), Pair(np.zeros_like(C23))
        getattr(r.cl, method)(c.cl, d.cl)
        O.apply(f"{stem}_3", [r.view, c.view, d.view])
        r.check(ulp, f"{method} out of place")


def test_atan2():
    c, d, r = Pair(C23), Pair(D23), Pair(np.zeros_like(C23))
    r.cl.atan2(c.cl, d.cl)
    O.apply("ATAN2_3", [r.view, c.view, d.view])
    r.check(2, "atan2")


@pytest.mark.parametrize("op", ["lt", "gt", "le", "ge", "eq", "ne"])
def test_compare(op):
    a, b = Pair(A23), Pair(B23)
    b.host[1] = a.host[1]  # one equal pair so that eq / le / ge see both outcomes
    b = Pair(b.host.reshape(2, 3))
    out = getattr(a.cl, op)(b.cl)
    r = Pair(np.zeros_like(A23))
    O.apply(f"{op.upper()}T_3", [r.view, a.view, b.view])
    assert np.array_equal(out.float(), r.view.numpy())
    out = getattr(a.cl, op)(2.0)
    O.apply(f"{op.upper()}V_2", [r.view, a.view], 2.0)
    assert np.array_equal(out.float(), r.view.numpy())


def test_scalar_ops_and_fills():
    p = Pair(A23)
    p.cl.add(1.5); O.apply("ADDC_1", [p.view], 1.5)
    p.cl.csub(0.25); O.apply("ADDC_1", [p.view], -0.25)
    p.cl.mul(3.0); O.apply("MULC_1", [p.view], 3.0)
    p.cl.div(7.0); O.apply("MULC_1", [p.view], np.float32(1.0) / np.float32(7.0))  # multiplies by 1/value
    p.check(0, "scalar chain")
    q = Pair(np.zeros((3, 2), np.float32))
    q.cl.fill(1.345); O.apply("FILL_1", [q.view], 1.345)
    q.check(0, "fill")
    q.cl.zero(); O.apply("FILL_1", [q.view], 0.0)
    q.check(0, "zero")


def test_clamp_pow_sign():
    p = Pair(A23)
    p.cl.clamp(1.5, 4.5); O.apply("CLAMP_1", [p.view], 1.5, 4.5)      # unit_tensor.lua:398-403
    p.check(0, "clamp")
    base = np.array([[3.3, -2.2, 0], [9, 7, 5]], np.float32)           # unit_tensor.lua:506-520
    with np.errstate(all="ignore"):
        p = Pair(base); p.cl.pow(2); O.apply("POWN_1", [p.view], 2.0); p.check(2, "integer power of a negative base")
        p = Pair(base); p.cl.pow(2.4); O.apply("POW_1", [p.view], 2.4); p.check(2, "fractional power (NaN for negative base)")


def test_cadd_with_scale_and_addcmul_addcdiv():
    a, b, c = (Pair(rng_uniform(s, (60, 50), -0.5, 0.5)) for s in (1, 2, 3))
    a.cl.add(1.234, b.cl); O.apply("CADD_2", [a.view, b.view], 1.234)
    a.check(0, "cadd")
    a.cl.addcmul(1.234, b.cl, c.cl); O.apply("ADDCMUL_3", [a.view, b.view, c.view], 1.234)   # unit_tensor.lua:539-546
    a.check(0, "addcmul")
    a.cl.addcdiv(1.234, b.cl, c.cl); O.apply("ADDCDIV_3", [a.view, b.view, c.view], 1.234)
    a.check(0, "addcdiv")
    # out-of-place form copies t into the result first; operands need equal counts, not shapes
    r, t = Pair(np.zeros(3000, np.float32)), Pair(rng_uniform(4, (3000,)))
    r.cl.addcmul(t.cl, 0.5, b.cl, c.cl)
    O.apply("COPY_2", [r.view, t.view]); O.apply("ADDCMUL_3", [r.view, b.view, c.view], 0.5)
    r.check(0, "addcmul out of place with differently shaped operands")


# ---- layouts ---------------------------------------------------------------------------------

def _layouts():
    """(name, storage shape, offset, sizes, strides): every one has 24*35 = 840 elements or so."""
    return [
        ("contiguous", (840,), 0, [24, 35], [35, 1]),
        ("offset-misaligned", (900,), 3, [24, 35], [35, 1]),
        ("transposed", (840,), 0, [24, 35], [1, 24]),
        ("narrow-cols", (24 * 50,), 7, [24, 35], [50, 1]),
        ("stride-2", (1700,), 1, [24, 35], [70, 2]),
        ("3d-permuted", (840,), 0, [4, 6, 35], [35, 140, 1]),
        ("unfold-like", (2000,), 0, [24, 35], [17, 3]),
    ]


@pytest.mark.parametrize("la,lb", list(itertools.product(range(7), range(7))))
def test_add_all_layout_pairs(la, lb):
    L = _layouts()
    _, sa, oa, za, ta = L[la]
    _, sb, ob, zb, tb = L[lb]
    if O.overlapping(za, ta):
        pytest.skip("destination overlaps itself")
    a = Pair(rng_uniform(5, sa, -1, 1), oa, za, ta)
    b = Pair(rng_uniform(6, sb, -1, 1), ob, zb, tb)
    c = Pair(rng_uniform(7, (840,), -1, 1))
    # in-place forms: the out-of-place ones resize the result like their first source
    a.cl.add(b.cl)
    O.apply("ADD_2", [a.view, b.view])
    a.check(0, f"{L[la][0]} += {L[lb][0]}")
    a.cl.addcmul(0.5, b.cl, c.cl)
    O.apply("ADDCMUL_3", [a.view, b.view, c.view], 0.5)
    a.check(0, f"{L[la][0]} += 0.5 * {L[lb][0]} * contiguous")
    b.check(0, "operand untouched")


@pytest.mark.parametrize("n", [0, 1, 2, 3, 4, 5, 7, 8, 15, 16, 17, 1023, 1024, 1025, 4099, 65537])
@pytest.mark.parametrize("offset", [0, 1, 2, 3])
def test_contiguous_ragged_sizes(n, offset):
    """Head/tail handling of the 128-bit kernel; guard elements around the view must survive."""
    a = Pair(rng_uniform(8, (n + 16,)), offset, [n] if n else [], None)
    b = Pair(rng_uniform(9, (n + 16,)), offset, [n] if n else [], None)
    if n == 0:
        a.cl.add(b.cl)          # zero elements: nothing happens
        a.check(0, "empty")
        return
    a.cl.cmul(b.cl); O.apply("MUL_2", [a.view, b.view])
    a.cl.add(2.5); O.apply("ADDC_1", [a.view], 2.5)
    a.check(0, f"n={n} offset={offset}")


@pytest.mark.parametrize("rows,cols,pitch", [(30, 28, 40), (257, 1028, 1200), (1, 8, 8), (70, 4, 12)])
def test_column_narrowed_views_take_the_row_vector_path(rows, cols, pitch):
    """R x C views with unit inner stride, 16-byte aligned rows and C % 4 == 0 (128-bit row kernel)."""
    import cltorch_b200 as cl
    a = Pair(rng_uniform(41, (rows * pitch + 8,), -1, 1), 4, [rows, cols], [pitch, 1])
    b = Pair(rng_uniform(42, (rows * pitch + 8,), -1, 1), 8, [rows, cols], [pitch, 1])
    c = Pair(rng_uniform(43, (rows * cols,), -1, 1), 0, [rows, cols], [cols, 1])
    a.cl.addcmul(0.5, b.cl, c.cl); O.apply("ADDCMUL_3", [a.view, b.view, c.view], 0.5)
    a.check(0, "narrowed += 0.5 * narrowed * contiguous")
    c.cl.add(a.cl); O.apply("ADD_2", [c.view, a.view])
    c.check(0, "contiguous += narrowed")
    a.cl.map_on_gpu(b.cl, "x = x * y + 0.25")
    want = O.eval_expr("x = x * y + 0.25", a.view.numpy(), b.view.numpy())
    a.view.numpy()[...] = want
    a.check(0, "expression on narrowed views")


@pytest.mark.parametrize("rows,cols", [(64, 32), (128, 96), (68, 36), (200, 132), (4, 4), (1028, 516)])
def test_transposed_operands_take_the_tile_path(rows, cols):
    """Transpose views with 16-byte friendly extents (128-bit tile kernel), destination row- or column-major."""
    import cltorch_b200 as cl
    n = rows * cols
    # contiguous (rows x cols) destination, two transposed sources
    a = Pair(rng_uniform(44, (n,), -1, 1), 0, [rows, cols], [cols, 1])
    b = Pair(rng_uniform(45, (n,), -1, 1), 0, [rows, cols], [1, rows])
    c = Pair(rng_uniform(46, (n,), -1, 1), 0, [rows, cols], [1, rows])
    a.cl.addcmul(0.5, b.cl, c.cl); O.apply("ADDCMUL_3", [a.view, b.view, c.view], 0.5)
    a.check(0, "row-major += 0.5 * transposed * transposed")
    # transposed destination
    b.cl.add(a.cl); O.apply("ADD_2", [b.view, a.view])
    b.check(0, "transposed += row-major")
    b.cl.addcmul(2.0, c.cl, a.cl); O.apply("ADDCMUL_3", [b.view, c.view, a.view], 2.0)
    b.check(0, "transposed += 2 * transposed * row-major")
    # write-only transposed destination through an expression
    b.cl.map_on_gpu(a.cl, "x = y * 3")
    b.view.numpy()[...] = a.view.numpy() * np.float32(3)
    b.check(0, "transposed = row-major * 3")
    a.check(0, "source untouched")


@pytest.mark.parametrize("rows,cols,pad", [(832, 768, 0), (1000, 1100, 0), (1028, 644, 8), (2048, 320, 4), (68, 9600, 0)])
def test_large_transposed_operands_go_through_the_tma_tiles(rows, cols, pad):
    """At least one 64 x 64 tile per SM: the tiles travel through the TMA unit (ragged edges are
    clipped by it). `pad` widens the pitch of every view beyond its extent."""
    prow, pcol = cols + pad, rows + pad
    a = Pair(rng_uniform(47, (rows * prow,), -1, 1), 0, [rows, cols], [prow, 1])      # row-major
    b = Pair(rng_uniform(48, (cols * pcol,), -1, 1), 0, [rows, cols], [1, pcol])      # column-major
    c = Pair(rng_uniform(49, (cols * pcol,), -1, 1), 0, [rows, cols], [1, pcol])
    d = Pair(rng_uniform(50, (rows * prow,), -1, 1), 0, [rows, cols], [prow, 1])
    a.cl.addcmul(0.5, b.cl, c.cl); O.apply("ADDCMUL_3", [a.view, b.view, c.view], 0.5)
    a.check(0, "row-major += 0.5 * transposed * transposed")
    b.cl.add(a.cl); O.apply("ADD_2", [b.view, a.view])
    b.check(0, "transposed += row-major")
    b.cl.addcmul(2.0, c.cl, a.cl); O.apply("ADDCMUL_3", [b.view, c.view, a.view], 2.0)
    b.check(0, "transposed += 2 * transposed * row-major")
    d.cl.add(b.cl, c.cl); O.apply("ADD_3", [d.view, b.view, c.view])                  # write-only destination
    d.check(0, "row-major = transposed + transposed")
    c.cl.cmul(a.cl, d.cl); O.apply("MUL_3", [c.view, a.view, d.view])
    c.check(0, "transposed = row-major * row-major")
    c.cl.copy(a.cl); O.apply("COPY_2", [c.view, a.view])
    c.check(0, "transposed = copy of row-major")
    d.cl.copy(b.cl); O.apply("COPY_2", [d.view, b.view])
    d.check(0, "row-major = copy of transposed")
    # run-time compiled expressions take the same kernel: one that reads its destination, one that does not
    want = O.eval_expr("x = x * y + z * 0.25", c.view.numpy(), a.view.numpy(), d.view.numpy())
    c.cl.map2_on_gpu(a.cl, d.cl, "x = x * y + z * 0.25")
    c.view.numpy()[...] = want
    c.check(0, "transposed = expression of itself and two row-major operands")
    want = O.eval_expr("x = y - 2 * z", d.view.numpy(), b.view.numpy(), c.view.numpy())
    d.cl.map2_on_gpu(b.cl, c.cl, "x = y - 2 * z")
    d.view.numpy()[...] = want
    d.check(0, "row-major = expression of two transposed operands")
    a.check(0, "sources untouched")
    b.cl.tanh(); O.apply("TANH_1", [b.view])                                          # last: 2 ulp of slack from here on
    b.check(2, "in place on a transposed view")


def test_mixed_alignment_falls_back_to_strided():
    a = Pair(rng_uniform(10, (5000,)), 1, [4000], None)
    b = Pair(rng_uniform(11, (5000,)), 2, [4000], None)
    a.cl.add(b.cl); O.apply("ADD_2", [a.view, b.view])
    a.check(0, "different 16-byte phases")


def test_overlapping_destination_goes_through_temporary():
    """An expanded (stride-0) read/write operand: contiguous temporary, then copy back
    (reference src/lib/THClApply.cpp:174-190). Every alias ends up holding one of the
    candidate results; with identical addends they all agree."""
    import cltorch_b200 as cl
    row = cl.ClTensor(np.array([[1.0, 2.0, 3.0]], np.float32))
    e = row.expand(4, 3)
    e.add(10.0)
    assert np.array_equal(row.float(), np.array([[11.0, 12.0, 13.0]], np.float32))


def test_copy_paths():
    import cltorch_b200 as cl
    base = rng_uniform(12, (60, 50))
    a = cl.ClTensor(base)
    assert np.array_equal(a.clone().float(), base)                       # contiguous: device memcpy
    assert np.array_equal(a.t().contiguous().float(), base.T)            # transposed: tile kernel
    assert np.array_equal(a.narrow(2, 10, 30).clone().float(), base[:, 9:39])
    assert np.array_equal(a.narrow(1, 10, 30).t().clone().float(), base[9:39].T)
    b = cl.ClTensor(50, 60)
    b.copy(a.t())
    assert np.array_equal(b.float(), base.T)
    c = cl.ClTensor(3000)
    c.copy(a)                                                            # equal counts, different shapes
    assert np.array_equal(c.float(), base.reshape(-1))
    d = cl.ClTensor(base.astype(np.float64))                             # typed host copies
    assert np.array_equal(d.double(), base.astype(np.float64))
    idx = cl.ClTensor(np.arange(12, dtype=np.int64).reshape(3, 4))
    assert np.array_equal(idx.long(), np.arange(12).reshape(3, 4))
    with pytest.raises(cl.ClError, match="sizes do not match"):
        c.copy(cl.ClTensor(7))


def test_element_access_and_storage():
    import cltorch_b200 as cl
    a = cl.ClTensor(np.arange(6, dtype=np.float32).reshape(2, 3))
    assert a[2, 3] == 5.0
    a[1, 2] = 42.0
    assert a.float()[0, 1] == 42.0
    s = cl.ClStorage(5).fill(1.5)
    s[2] = 9.0
    assert list(s.float()) == [1.5, 9.0, 1.5, 1.5, 1.5]
    with pytest.raises(cl.ClError, match="out of"):
        a[3, 1]


# ---- user expressions (apply_on_gpu / map_on_gpu / map2_on_gpu) ------------------------------------

def test_apply_on_gpu_both_spellings():
    A = rng_uniform(13, (6, 4), -0.5, 0.5)                                # unit_tensor.lua:583-592
    want = O.eval_expr("x = sqrt(x + 3) + exp(x)", A)
    import cltorch_b200 as cl
    got1 = cl.ClTensor(A).apply_on_gpu("*out = sqrt(*out + 3) + exp(*out)").float()
    got2 = cl.ClTensor(A).apply_on_gpu("x = sqrt(x + 3) + exp(x)").float()
    assert np.array_equal(got1, got2)
    assert O.ulp_diff(got1, want).max() <= 2


def test_map_and_map2_on_gpu():
    import cltorch_b200 as cl
    A, B, Cc = (rng_uniform(s, (60, 50), -0.5, 0.5) for s in (14, 15, 16))
    want = O.eval_expr("x = sqrt(x * x + y * y + 3 + exp(y))", A, B)      # unit_tensor.lua:594-610
    got = cl.ClTensor(A).map_on_gpu(cl.ClTensor(B), "x = sqrt(x * x + y * y + 3 + exp(y))").float()
    assert O.ulp_diff(got, want).max() <= 2
    got = cl.ClTensor(A).apply2_on_gpu(cl.ClTensor(B), "*out = sqrt(*out * *out + *in1 * *in1 + 3 + exp(*in1))").float()
    assert O.ulp_diff(got, want).max() <= 2
    want = O.eval_expr("x = sqrt(x * x + y * y + z + 3 + exp(z))", A, B, Cc)   # unit_tensor.lua:612-635
    got = cl.ClTensor(A).map2_on_gpu(cl.ClTensor(B), cl.ClTensor(Cc), "x = sqrt(x * x + y * y + z + 3 + exp(z))").float()
    assert O.ulp_diff(got, want).max() <= 2


def test_readme_expressions():
    import cltorch_b200 as cl
    x, y, z = (rng_uniform(s, (40, 30)) for s in (17, 18, 19))
    for nt, expr in [(1, "x = sqrt(x + 3.5)"), (2, "x = 1000 * x + y * 10"), (3, "x = sqrt(1000 * x + y * 10 + z * z)")]:
        args = [cl.ClTensor(v) for v in (x, y, z)[:nt]]
        want = O.eval_expr(expr, *(x, y, z)[:nt])
        if nt == 1:
            got = args[0].apply_on_gpu(expr)
        elif nt == 2:
            got = args[0].map_on_gpu(args[1], expr)
        else:
            got = args[0].map2_on_gpu(args[1], args[2], expr)
        assert np.array_equal(got.float(), want), expr   # + * sqrt only: exactly rounded on both sides


def test_expression_on_strided_operands_and_identifiers():
    import cltorch_b200 as cl
    base = rng_uniform(20, (64, 48), -1, 1)
    a = cl.ClTensor(base)
    out = cl.ClTensor(48, 64).zero()
    out.map_on_gpu(a.t(), "x = max(y, 0.25) * exp(y)")       # identifiers containing x/y must survive
    want = O.eval_expr("x = max(y, 0.25) * exp(y)", np.zeros((48, 64), np.float32), base.T)
    assert O.ulp_diff(out.float(), want).max() <= 2


@pytest.mark.parametrize("expr", ["if (y > 0) x = y", "if (y > 0) { x = y; }", "for (int i = 0; i < 2; ++i) if (y > i) x = y + i"])
def test_expression_with_conditional_store_keeps_other_elements(expr):
    """A body that stores only under a condition must leave every other element as it was (the reference
    hands the operator a pointer into the tensor). Contiguous, stride-2, small transposed (tile kernel) and
    large transposed (TMA tile kernel) layouts."""
    import cltorch_b200 as cl

    def want(x, y):
        if expr.startswith("for"):
            out = np.where(y > 0, y, x)
            return np.where(y > 1, y + np.float32(1), out).astype(np.float32)
        return np.where(y > 0, y, x).astype(np.float32)

    g = np.random.Generator(np.random.PCG64(77))
    # contiguous, with a ragged length so that the scalar head / tail run too
    x, y = (g.uniform(-2, 2, 100003).astype(np.float32) for _ in range(2))
    got = cl.ClTensor(x).map_on_gpu(cl.ClTensor(y), expr).float()
    assert np.array_equal(got, want(x, y)), "contiguous"
    # every second element of the destination; the elements in between must not change either
    base = g.uniform(-2, 2, 20000).astype(np.float32)
    full = cl.ClTensor(base)
    view = cl.ClTensor(full.storage(), 1, [10000], [2])
    yy = g.uniform(-2, 2, 10000).astype(np.float32)
    view.map_on_gpu(cl.ClTensor(yy), expr)
    expect = base.copy()
    expect[::2] = want(base[::2], yy)
    assert np.array_equal(full.float(), expect), "stride 2"
    # transposed source: a small matrix and one large enough for a tile per SM
    for rows, cols in ((96, 80), (1024, 1536)):
        xs = g.uniform(-2, 2, (rows, cols)).astype(np.float32)
        ys = g.uniform(-2, 2, (cols, rows)).astype(np.float32)
        got = cl.ClTensor(xs).map_on_gpu(cl.ClTensor(ys).t(), expr).float()
        assert np.array_equal(got, want(xs, ys.T)), f"transposed {rows}x{cols}"
        out = cl.ClTensor(ys.copy())
        out.t().map_on_gpu(cl.ClTensor(xs), expr)                # transposed destination
        assert np.array_equal(out.float(), want(ys.T, xs).T), f"transposed destination {rows}x{cols}"


def test_expression_errors_are_reported():
    import cltorch_b200 as cl
    a = cl.ClTensor(np.ones(4, np.float32))
    with pytest.raises(cl.ClError, match="did not compile"):
        a.apply_on_gpu("x = nosuchfunction(x)")
    with pytest.raises(cl.ClError, match="element size mismatch"):
        a.map_on_gpu(cl.ClTensor(np.ones(5, np.float32)), "x = y")
    assert np.array_equal(a.float(), np.ones(4, np.float32))   # the library is still usable


def test_large_chain_walks_the_operands_from_either_end():
    """Operands larger than L2: a contiguous apply starts at the end that the previous kernel left in
    L2, so every second kernel of a chain walks its batches downwards. The order in time must not show
    in any result, ragged head and tail included."""
    import cltorch_b200 as cl
    n = (1 << 26) + 5
    base = rng_uniform(77, (n + 3,), 0.0, 4.0)
    for offset in (0, 3):                                                 # 16-byte aligned / three elements off
        host = base[offset:offset + n]
        x = cl.ClTensor(cl.ClStorage(base.copy()), offset + 1, [n], [1])
        y = cl.ClTensor(host * np.float32(0.5))
        want = host.copy()
        for _ in range(2):                                                # four applies in a row over the same memory
            x.apply_on_gpu("x = x * 1.0001 + 0.5"); want = want * np.float32(1.0001) + np.float32(0.5)
            x.map_on_gpu(y, "x = sqrt(x + y)"); want = np.sqrt(want + host * np.float32(0.5))
        assert np.array_equal(x.float(), want)
        assert abs(x.sum() - float(want.astype(np.float64).sum())) <= 1e-6 * float(want.astype(np.float64).sum())


def test_asynchronous_upload_on_a_second_stream():
    """THClTensor_copyFloatAsync: the upload is enqueued on a stream of the caller's and ordered against the
    library's stream by the caller's events."""
    import torch
    import cltorch_b200 as cl
    n = 1 << 22
    host = torch.empty(n, dtype=torch.float32, pin_memory=True)
    hv = host.numpy()
    hv[:] = rng_uniform(78, (n,), 0.0, 2.0)
    compute, copy = torch.cuda.ExternalStream(cl.getStream()), torch.cuda.Stream()   # the library's stream, a second one
    t = cl.ClTensor(n).fill(-1.0)
    cl.synchronize()
    t.copy_async(hv, copy.cuda_stream)
    done = torch.cuda.Event()
    done.record(copy)
    compute.wait_event(done)
    t.mul(2.0)
    assert np.array_equal(t.float(), hv * np.float32(2.0))
    with pytest.raises(cl.ClError, match="sizes do not match"):
        cl.ClTensor(5).copy_async(hv)
    with pytest.raises(cl.ClError, match="contiguous"):
        cl.ClTensor(n // 2, 2).t().copy_async(hv)
