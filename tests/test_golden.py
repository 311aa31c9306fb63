"""The known answers implied by the reference's own tests (tests/golden/), checked twice:
against the CPU oracle (this pins the oracle; runs without a GPU) and against the CUDA
path through the THCl C API (marked gpu). Tolerances are the ones stored with each case:
0 where the answer is exactly representable, else the 2e-4 the reference's tests use.
"""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O

GOLD = json.loads((Path(__file__).parent / "golden" / "reference_known_answers.json").read_text())
CASES = GOLD["cases"]


def _expected(case):
    vals = [np.nan if v is None else (np.inf if v == "inf" else (-np.inf if v == "-inf" else v)) for v in case["expected"]]
    return np.array(vals, dtype=np.float64).reshape(case["shape"])


def _uniform(seed, shape):
    g = np.random.Generator(np.random.PCG64(seed))
    return (g.random(shape, dtype=np.float32) + np.float32(-0.5)).astype(np.float32)


def _views(name, arr):
    return {"t": arr.T, "narrow1_t": arr[9:39].T, "narrow2_t": arr[:, 9:39].T}[name]


UNARY_STEM = {"abs": "ABS", "sqrt": "SQRT", "log": "LOG", "exp": "EXP", "cos": "COS", "acos": "ACOS", "sin": "SIN",
              "asin": "ASIN", "atan": "ATAN", "tanh": "TANH", "ceil": "CEIL", "floor": "FLOOR", "round": "ROUND",
              "sign": "SIGN", "sigmoid": "SIGMOID", "cinv": "CINV", "neg": "NEG"}
BINARY_STEM = {"add": "ADD", "cmul": "MUL", "cdiv": "DIV", "cpow": "CPOW", "atan2": "ATAN2", "csub": "SUB"}


def run_oracle(case):
    op, inp = case["op"], case["inputs"]
    f = lambda k: np.array(inp[k], dtype=np.float32)
    with np.errstate(all="ignore"):
        if op in UNARY_STEM:
            a = f("a"); O.apply(UNARY_STEM[op] + "_1", [O.View(a)]); return a
        if op in BINARY_STEM:
            a, b = f("a"), f("b"); O.apply(BINARY_STEM[op] + "_2", [O.View(a), O.View(b)]); return a
        if op in ("lt", "gt", "le", "ge", "eq", "ne"):
            a, b, r = f("a"), f("b"), np.zeros_like(f("a"))
            O.apply(op.upper() + "T_3", [O.View(r), O.View(a), O.View(b)]); return r
        if op == "clamp":
            a = f("a"); O.apply("CLAMP_1", [O.View(a)], inp["lo"], inp["hi"]); return a
        if op == "pow":
            a = f("a"); v = inp["v"]
            O.apply("POWN_1" if float(int(v)) == v else "POW_1", [O.View(a)], v); return a
        if op == "fill":
            a = np.zeros(inp["shape"], np.float32); O.apply("FILL_1", [O.View(a)], inp["v"]); return a
        if op in ("maxall", "minall", "sumall"):
            a = f("a") if "a" in inp else _uniform(inp["seed"], inp["shape"])
            red, init = {"maxall": ("max", -np.inf), "minall": ("min", np.inf), "sumall": ("add", 0.0)}[op]
            return np.array([O.reduce_all(O.View(a), red=red, init=init)])
        if op == "sum":
            return O.reduce_dim(O.View(f("a")), inp["dim"])
        if op == "sum_view":
            return O.reduce_dim(O.View.of(_views(inp["view"], _uniform(inp["seed"], inp["shape"]))), inp["dim"])
        if op == "mm":
            a, b = f("a"), f("b")
            return O.addmm(0.0, np.zeros((a.shape[0], b.shape[1]), np.float32), 1.0, a, b)
        if op == "apply":
            x = _uniform(inp["seed"], inp["shape"])
            r1, r2 = O.eval_expr(inp["expr"], x), O.eval_expr(inp["expr_raw"], x)
            assert np.array_equal(r1, r2)
            return r1
        if op in ("map", "map2"):
            arrs = [_uniform(s, inp["shape"]) for s in inp["seed"]]
            return O.eval_expr(inp["expr"], *arrs)
        if op in ("addcmul", "addcdiv"):
            a, b, c = (_uniform(s, inp["shape"]) for s in inp["seed"])
            O.apply(op.upper() + "_3", [O.View(a), O.View(b), O.View(c)], inp["v"]); return a
        if op in ("max", "min"):
            return O.reduce_dim_index(f("a"), inp["dim"], op == "max")
        if op in ("cumsum", "cumprod"):
            a = f("a") if "a" in inp else _uniform(inp["seed"], inp["shape"])
            return O.scan(a, inp["dim"], op == "cumprod")
        if op in ("var", "std"):
            return O.var_dim(f("a"), inp["dim"], inp["flag"], op == "std")
        if op in ("varall", "stdall"):
            return O.var_dim(f("a").reshape(1, -1), 1, False, op == "stdall").reshape(1)
        if op == "renorm":
            return O.renorm(f("a"), inp["p"], inp["dim"], inp["maxnorm"])
        if op == "dist":
            return np.array([O.dist(f("a"), f("b"), inp["p"])])
    raise AssertionError(f"no oracle runner for {op}")


def run_gpu(case):
    import cltorch_b200 as cl
    op, inp = case["op"], case["inputs"]
    T = lambda k: cl.ClTensor(np.array(inp[k], dtype=np.float32))
    if op in UNARY_STEM:
        return getattr(T("a"), op)().float()
    if op in BINARY_STEM:
        return getattr(T("a"), op)(T("b")).float()
    if op in ("lt", "gt", "le", "ge", "eq", "ne"):
        return getattr(T("a"), op)(T("b")).float()
    if op == "clamp":
        return T("a").clamp(inp["lo"], inp["hi"]).float()
    if op == "pow":
        return T("a").pow(inp["v"]).float()
    if op == "fill":
        return cl.ClTensor(*inp["shape"]).fill(inp["v"]).float()
    if op in ("maxall", "minall", "sumall"):
        a = T("a") if "a" in inp else cl.ClTensor(_uniform(inp["seed"], inp["shape"]))
        return np.array([{"maxall": a.max, "minall": a.min, "sumall": a.sum}[op]()])
    if op == "sum":
        return T("a").sum(inp["dim"] + 1).float()
    if op == "sum_view":
        A = cl.ClTensor(_uniform(inp["seed"], inp["shape"]))
        v = {"t": lambda: A.t(), "narrow1_t": lambda: A.narrow(1, 10, 30).t(), "narrow2_t": lambda: A.narrow(2, 10, 30).t()}[inp["view"]]()
        return v.sum(inp["dim"] + 1).float()
    if op == "mm":
        return cl.ClTensor().mm(T("a"), T("b")).float()
    if op == "apply":
        x = _uniform(inp["seed"], inp["shape"])
        r1 = cl.ClTensor(x).apply_on_gpu(inp["expr"]).float()
        r2 = cl.ClTensor(x).apply_on_gpu(inp["expr_raw"]).float()
        assert np.array_equal(r1, r2)
        return r1
    if op in ("map", "map2"):
        ts = [cl.ClTensor(_uniform(s, inp["shape"])) for s in inp["seed"]]
        return (ts[0].map_on_gpu(ts[1], inp["expr"]) if op == "map" else ts[0].map2_on_gpu(ts[1], ts[2], inp["expr"])).float()
    if op in ("addcmul", "addcdiv"):
        a, b, c = (cl.ClTensor(_uniform(s, inp["shape"])) for s in inp["seed"])
        return getattr(a, op)(inp["v"], b, c).float()
    if op in ("max", "min"):
        v, i = getattr(T("a"), op)(inp["dim"] + 1)
        return v.float(), i.float()
    if op in ("cumsum", "cumprod"):
        a = T("a") if "a" in inp else cl.ClTensor(_uniform(inp["seed"], inp["shape"]))
        return getattr(a, op)(inp["dim"] + 1).float()
    if op in ("var", "std"):
        return getattr(T("a"), op)(inp["dim"] + 1, inp["flag"]).float()
    if op in ("varall", "stdall"):
        return np.array([getattr(T("a"), op[:3])()])
    if op == "renorm":
        return T("a").renorm(inp["p"], inp["dim"] + 1, inp["maxnorm"]).float()
    if op == "dist":
        return np.array([T("a").dist(T("b"), inp["p"])])
    raise AssertionError(f"no GPU runner for {op}")


def _check(case, got):
    want = _expected(case)
    if case["op"] in ("max", "min"):
        values, indices = got
        assert np.array_equal(np.asarray(values, dtype=np.float64), want)
        want_i = np.array(case["indices"], dtype=np.float64).reshape(case["shape"])
        assert np.array_equal(np.asarray(indices, dtype=np.float64), want_i)
        return
    got = np.asarray(got, dtype=np.float64).reshape(want.shape)
    assert np.array_equal(np.isnan(got), np.isnan(want)), f"{case['name']}: NaN pattern differs"
    ok = ~np.isnan(want)
    err = np.abs(got[ok] - want[ok])
    err = np.where(np.isinf(want[ok]) & (got[ok] == want[ok]), 0.0, err)
    assert err.size == 0 or err.max() <= case["tol"], f"{case['name']} ({case['source']}): max error {err.max()} > {case['tol']}"


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_known_answers(case):
    _check(case, run_oracle(case))


@pytest.mark.parametrize("c", GOLD["collapse"], ids=[f"collapse{k}" for k in range(len(GOLD["collapse"]))])
def test_oracle_collapse_matches_hand_worked_cases(c):
    assert O.collapse(c["size"], c["stride"], c["reduce_dim"]) == (c["out_size"], c["out_stride"])


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_gpu_matches_known_answers(case):
    _check(case, run_gpu(case))
