"""Generates tests/golden/reference_known_answers.json.

The reference (hughperkins/cltorch) cannot be run here, and its test-suite stores almost no
outputs: each test builds a small ClTensor, runs the same method on a Torch7 CPU tensor
and compares within 2e-4 (Float) / 1e-4 (Double) (src/test/unit_tensor.lua:73-115). What
this script records is therefore the *answer those tests imply*: the literal inputs of the
reference's tests (or seeded stand-ins where the test draws random numbers), and the
expected output computed here in float64 from the mathematical definition the test
uses, independently of both the CUDA library and the oracle. Cases whose result is
exactly representable carry tol = 0.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
from pathlib import Path

import numpy as np

OUT = Path(__file__).resolve().parent / "reference_known_answers.json"

A23 = [[4, 2, -1], [3.1, 1.2, 4.9]]      # unit_tensor.lua:225-228, 239-240
B23 = [[3, 5, -2], [2.1, 2.2, 3.9]]
C23 = [[4, 2, -1], [0.8, 1.2, 1.9]]      # unit_tensor.lua:267-270
D23 = [[3, 5, -2], [2.1, 2.2, 0.9]]
M23 = [[3, 2, 4], [9, 7, 5]]             # unit_tensor.lua:489
P23 = [[3.3, -2.2, 0], [9, 7, 5]]        # unit_tensor.lua:507, 515
TOL = 2e-4                               # torch.FloatTensor.__eq, unit_tensor.lua:73-92


def f32(a):
    return np.asarray(a, dtype=np.float32)


def lst(a):
    a = np.asarray(a, dtype=np.float64)
    return [None if np.isnan(v) else (float(v) if np.isfinite(v) else ("inf" if v > 0 else "-inf")) for v in a.ravel()]


def uniform(seed, shape, shift=-0.5):
    g = np.random.Generator(np.random.PCG64(seed))
    return (g.random(shape, dtype=np.float32) + np.float32(shift)).astype(np.float32)


cases = []


def case(name, source, op, inputs, expected, tol, **extra):
    cases.append(dict(name=name, source=source, op=op, inputs=inputs, expected=lst(expected),
                      shape=list(np.asarray(expected).shape), tol=tol, **extra))


with np.errstate(all="ignore"):
    a = f32(A23).astype(np.float64)
    unary = {
        "abs": (np.abs, 0), "sqrt": (np.sqrt, TOL), "log": (np.log, TOL), "exp": (np.exp, TOL), "cos": (np.cos, TOL),
        "acos": (np.arccos, TOL), "sin": (np.sin, TOL), "asin": (np.arcsin, TOL), "atan": (np.arctan, TOL),
        "tanh": (np.tanh, TOL), "ceil": (np.ceil, 0), "floor": (np.floor, 0),
        "round": (lambda v: np.sign(v) * np.floor(np.abs(v) + 0.5), 0), "sign": (np.sign, 0),
        "sigmoid": (lambda v: 1 / (1 + np.exp(-v)), TOL), "cinv": (lambda v: 1 / v, TOL), "neg": (lambda v: -v, 0),
    }
    for name, (fn, tol) in unary.items():
        case(f"unary_{name}", "src/test/unit_tensor.lua:237-263", name, {"a": A23}, fn(a), tol)

    c, d = f32(C23).astype(np.float64), f32(D23).astype(np.float64)
    binary = {"add": c + d, "cmul": c * d, "cdiv": c / d, "cpow": np.power(c, d), "atan2": np.arctan2(c, d),
              "csub": c - d}
    for name, want in binary.items():
        case(f"binary_{name}", "src/test/unit_tensor.lua:265-307", name, {"a": C23, "b": D23}, want, TOL)

    a2, b2 = f32(A23), f32(B23)
    for name, fn in {"lt": np.less, "gt": np.greater, "le": np.less_equal, "ge": np.greater_equal,
                     "eq": np.equal, "ne": np.not_equal}.items():
        case(f"compare_{name}", "src/test/unit_tensor.lua:222-235,280-292", name, {"a": A23, "b": B23},
             fn(a2, b2).astype(np.float64), 0)

    case("clamp", "src/test/unit_tensor.lua:398-403", "clamp", {"a": A23, "lo": 1.5, "hi": 4.5}, np.clip(a, 1.5, 4.5), 0)
    case("pow_int", "src/test/unit_tensor.lua:506-512", "pow", {"a": P23, "v": 2}, f32(P23).astype(np.float64) ** 2, TOL)
    case("pow_frac", "src/test/unit_tensor.lua:514-520", "pow", {"a": P23, "v": 2.4},
         np.power(f32(P23).astype(np.float64), 2.4), TOL)
    case("fill", "src/test/unit_tensor.lua:463-468", "fill", {"shape": [3, 2], "v": 1.345},
         np.full((3, 2), np.float64(np.float32(1.345))), 0)

    m = f32(M23).astype(np.float64)
    case("max_all", "src/test/unit_tensor.lua:488-496", "maxall", {"a": M23}, [m.max()], 0)
    case("min_all", "src/test/unit_tensor.lua:488-496", "minall", {"a": M23}, [m.min()], 0)
    case("sum_all", "src/test/unit_tensor.lua:488-496", "sumall", {"a": M23}, [m.sum()], 0)
    case("sum_dim1", "src/test/unit_tensor.lua:488-496", "sum", {"a": M23, "dim": 0}, m.sum(axis=0, keepdims=True), 0)
    case("sum_dim2", "src/test/unit_tensor.lua:488-496", "sum", {"a": M23, "dim": 1}, m.sum(axis=1, keepdims=True), 0)
    case("mm", "src/test/unit_tensor.lua:413-425", "mm", {"a": [[1, 2, -1], [3, 4, 0]], "b": [[0, 1], [1, 2], [4, 5]]},
         np.array([[1, 2, -1], [3, 4, 0]], dtype=np.float64) @ np.array([[0, 1], [1, 2], [4, 5]], dtype=np.float64), 0)

    # user expressions: the Lua tests evaluate the same formula with math.* in doubles
    A = uniform(101, (6, 4))
    case("apply_on_gpu", "src/test/unit_tensor.lua:583-592", "apply", {"seed": 101, "shape": [6, 4],
         "expr": "x = sqrt(x + 3) + exp(x)", "expr_raw": "*out = sqrt(*out + 3) + exp(*out)"},
         np.sqrt(A.astype(np.float64) + 3) + np.exp(A.astype(np.float64)), TOL)
    A, B = uniform(102, (60, 50)), uniform(103, (60, 50))
    A64, B64 = A.astype(np.float64), B.astype(np.float64)
    case("map_on_gpu", "src/test/unit_tensor.lua:594-610", "map", {"seed": [102, 103], "shape": [60, 50],
         "expr": "x = sqrt(x * x + y * y + 3 + exp(y))"}, np.sqrt(A64 * A64 + B64 * B64 + 3 + np.exp(B64)), TOL)
    Cc = uniform(104, (60, 50))
    C64 = Cc.astype(np.float64)
    case("map2_on_gpu", "src/test/unit_tensor.lua:612-635", "map2", {"seed": [102, 103, 104], "shape": [60, 50],
         "expr": "x = sqrt(x * x + y * y + z + 3 + exp(z))"}, np.sqrt(A64 * A64 + B64 * B64 + C64 + 3 + np.exp(C64)), TOL)
    case("addcmul", "src/test/unit_tensor.lua:539-546", "addcmul", {"seed": [102, 103, 104], "shape": [60, 50], "v": 1.234},
         A64 + np.float64(np.float32(1.234)) * B64 * C64, TOL)
    case("addcdiv", "src/test/unit_tensor.lua:548-556", "addcdiv", {"seed": [102, 103, 104], "shape": [60, 50], "v": 1.234},
         A64 + np.float64(np.float32(1.234)) * B64 / C64, TOL * 50)  # quotients by small |c| amplify fp32 rounding

    # two-pass reduceAll on ~10M elements; the reference accepts |diff| < 1.2 (unit_tensor.lua:637-646)
    big = uniform(105, (28 * 28 * 1280, 10))
    case("reduce_all_two_pass", "src/test/unit_tensor.lua:637-646", "sumall", {"seed": 105, "shape": [28 * 28 * 1280, 10]},
         [big.sum(dtype=np.float64)], 1.2)
    small = uniform(106, (50, 40))
    case("reduce_all_one_pass", "src/test/unit_tensor.lua:648-656", "sumall", {"seed": 106, "shape": [50, 40]},
         [small.sum(dtype=np.float64)], 0.1)

    # sums of narrowed + transposed views (Lua 1-based narrow(1,10,30) = rows 9..38)
    S = uniform(107, (60, 50))
    for vname, view in {"t": S.T, "narrow1_t": S[9:39].T, "narrow2_t": S[:, 9:39].T}.items():
        for dim in (0, 1):
            case(f"sum_{vname}_dim{dim + 1}", "src/test/unit_tensor.lua:759-775", "sum_view",
                 {"seed": 107, "shape": [60, 50], "view": vname, "dim": dim},
                 view.astype(np.float64).sum(axis=dim, keepdims=True), TOL)

    # max / min with 1-based indices (unit_tensor.lua:786-832); fixed values with ties
    Mx = [[0.25, -0.5], [0.75, 0.125], [0.75, -0.5], [-0.25, 0.125], [0.5, 0.0]]
    mx = np.array(Mx)
    for dim in (0, 1):
        case(f"max_dim{dim + 1}", "src/test/unit_tensor.lua:786-808", "max", {"a": Mx, "dim": dim},
             mx.max(axis=dim, keepdims=True), 0, indices=lst(np.expand_dims(mx.argmax(axis=dim) + 1, dim)))
        case(f"min_dim{dim + 1}", "src/test/unit_tensor.lua:810-832", "min", {"a": Mx, "dim": dim},
             mx.min(axis=dim, keepdims=True), 0, indices=lst(np.expand_dims(mx.argmin(axis=dim) + 1, dim)))

    # scans: the literal matrix of src/test/test-tensor.lua:612-626 (exact), and the seeded 50 x 60 of
    # src/test/unit_tensor.lua:876-888 (default dimension = first, src/TensorMath.lua:955-961)
    Asc = [[3, 1, 7], [3, 2, 4]]
    asc = np.array(Asc, dtype=np.float64)
    for dim in (0, 1):
        case(f"cumsum_dim{dim + 1}", "src/test/test-tensor.lua:612-617", "cumsum", {"a": Asc, "dim": dim}, np.cumsum(asc, axis=dim), 0)
        case(f"cumprod_dim{dim + 1}", "src/test/test-tensor.lua:619-626", "cumprod", {"a": Asc, "dim": dim}, np.cumprod(asc, axis=dim), 0)
    X = uniform(108, (50, 60))
    for dim in (0, 1):
        case(f"cumsum_uniform_dim{dim + 1}", "src/test/unit_tensor.lua:876-881", "cumsum", {"seed": 108, "shape": [50, 60], "dim": dim},
             np.cumsum(X.astype(np.float64), axis=dim), TOL)
        case(f"cumprod_uniform_dim{dim + 1}", "src/test/unit_tensor.lua:883-888", "cumprod", {"seed": 108, "shape": [50, 60], "dim": dim},
             np.cumprod(X.astype(np.float64), axis=dim), TOL)

    # var / std along a dimension: THClTensor_computeVar, src/lib/THClTensorMath2.cl:5-23 (flag: divide by n)
    for dim in (0, 1):
        for flag in (False, True):
            case(f"var_dim{dim + 1}_flag{int(flag)}", "src/lib/THClTensorMath2.cl:5-23", "var", {"a": M23, "dim": dim, "flag": flag},
                 m.var(axis=dim, ddof=0 if flag else 1, keepdims=True), 1e-6)
            case(f"std_dim{dim + 1}_flag{int(flag)}", "src/lib/THClTensorMath2.cl:5-23", "std", {"a": M23, "dim": dim, "flag": flag},
                 m.std(axis=dim, ddof=0 if flag else 1, keepdims=True), 1e-6)
    case("var_all", "src/lib/THClTensorMath2.cpp:209-223", "varall", {"a": M23}, [m.var(ddof=1)], 1e-6)
    case("std_all", "src/lib/THClTensorMath2.cpp:225-229", "stdall", {"a": M23}, [m.std(ddof=1)], 1e-6)

    # renorm (src/lib/THClTensorMath2.cl:110-143): rows of norm > maxnorm scaled by maxnorm / (norm + 1e-7)
    R = [[3, 4, 0], [0.3, 0.4, 0], [1, 2, 2]]                     # 2-norms of the rows: 5, 0.5, 3
    r = np.array(R, dtype=np.float64)
    nr = np.sqrt((r * r).sum(axis=1, keepdims=True))
    case("renorm_rows", "src/lib/THClTensorMath2.cl:110-143", "renorm", {"a": R, "p": 2, "dim": 0, "maxnorm": 1},
         np.where(nr > 1, r * (1 / (nr + 1e-7)), r), 1e-6)
    nc = np.abs(r).sum(axis=0, keepdims=True)                      # 1-norms of the columns: 4.3, 6.4, 2
    case("renorm_cols", "src/lib/THClTensorMath2.cl:110-143", "renorm", {"a": R, "p": 1, "dim": 1, "maxnorm": 3},
         np.where(nc > 3, r * (3 / (nc + 1e-7)), r), 1e-6)

    # dist (src/lib/THClTensorMath2.cpp:448-475)
    cd, dd = f32(C23).astype(np.float64), f32(D23).astype(np.float64)
    for pv in (1, 2, 3):
        case(f"dist_p{pv}", "src/lib/THClTensorMath2.cpp:448-475", "dist", {"a": C23, "b": D23, "p": pv},
             [(np.abs(cd - dd) ** pv).sum() ** (1.0 / pv)], 1e-5)

# Dimension collapsing (src/lib/THClReduceApplyUtils.h:68-170), worked by hand from the rule
# "drop size-1 dims; merge dim i into i+1 when stride[i] == size[i+1]*stride[i+1]".
collapse = [
    dict(size=[4, 5, 6], stride=[30, 6, 1], reduce_dim=-1, out_size=[120], out_stride=[1]),
    dict(size=[5, 4], stride=[1, 5], reduce_dim=-1, out_size=[5, 4], out_stride=[1, 5]),
    dict(size=[8192, 4096], stride=[8192, 2], reduce_dim=-1, out_size=[33554432], out_stride=[2]),
    dict(size=[4000, 8192], stride=[8192, 1], reduce_dim=-1, out_size=[32768000], out_stride=[1]),
    dict(size=[8192, 4000], stride=[8192, 1], reduce_dim=-1, out_size=[8192, 4000], out_stride=[8192, 1]),
    dict(size=[1, 1, 1], stride=[7, 3, 1], reduce_dim=-1, out_size=[1], out_stride=[1]),
    dict(size=[3, 1, 5], stride=[5, 99, 1], reduce_dim=-1, out_size=[15], out_stride=[1]),
    dict(size=[4, 5, 6], stride=[30, 6, 1], reduce_dim=1, out_size=[4, 6], out_stride=[30, 1]),
    dict(size=[4, 5, 6], stride=[30, 6, 1], reduce_dim=2, out_size=[20], out_stride=[6]),
    dict(size=[4, 5, 6], stride=[30, 6, 1], reduce_dim=0, out_size=[30], out_stride=[1]),
    dict(size=[2, 3, 4, 5], stride=[60, 20, 5, 1], reduce_dim=-1, out_size=[120], out_stride=[1]),
    dict(size=[2, 3, 4, 5], stride=[120, 20, 5, 1], reduce_dim=-1, out_size=[2, 60], out_stride=[120, 1]),
    dict(size=[2, 3, 4, 5], stride=[60, 20, 1, 4], reduce_dim=-1, out_size=[6, 4, 5], out_stride=[20, 1, 4]),
    dict(size=[6, 4], stride=[0, 1], reduce_dim=-1, out_size=[6, 4], out_stride=[0, 1]),
]

OUT.write_text(json.dumps({"cases": cases, "collapse": collapse}, indent=1))
print(f"wrote {OUT} ({len(cases)} cases, {len(collapse)} collapse cases)")
