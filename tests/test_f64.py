"""Float64 on the device.  Most of Reactant's own tests run on Float64 arrays (test/core/map_reduction.jl:8-19); a
fusion group that touches an f64 value is lowered as a "wide" program and runs on the 64-bit-register interpreter
kernels.  CPU: every f64 fixture plans, its groups are flagged wide, and f64 never shares a group with 32-bit floats.
GPU: the 13 f64 fixtures restated from the reference's tests against their exact expectations (1e-12), and
elementwise / reduction / scan / dot_general programs against the numpy oracle (which computes f64 as float64)."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reactant_fixtures.json")) as f:
    F64_CASES = [c for c in json.load(f)["cases"] if c["element_type"] == "f64"]


def steps_of(plan):
    out = []
    for s in plan["steps"]:
        out.append(s)
        out += steps_of({"steps": s.get("body", [])})
    return out


def test_every_f64_fixture_plans_as_wide_programs(rx):
    assert len(F64_CASES) == 13
    for c in F64_CASES:
        p = rx.plan_describe(c["module"])
        chains = [s for s in steps_of(p) if "chain" in s]
        assert all(s.get("wide") == 1 for s in chains), (c["name"], p)


def test_f64_and_f32_do_not_share_a_group(rx):
    t32, t64 = "tensor<64x64xf32>", "tensor<64x64xf64>"
    text = f"""module {{
  func.func @main(%arg0: {t32}, %arg1: {t64}) -> ({t64}, {t32}) {{
    %0 = stablehlo.sine %arg0 : {t32}
    %1 = stablehlo.convert %0 : ({t32}) -> {t64}
    %2 = stablehlo.multiply %1, %arg1 : {t64}
    %3 = stablehlo.convert %2 : ({t64}) -> {t32}
    %4 = stablehlo.cosine %3 : {t32}
    return %2, %4 : {t64}, {t32}
  }}
}}
"""
    p = rx.plan_describe(text)
    chains = [s for s in p["steps"] if "chain" in s]
    # sin in f32 (narrow), multiply in f64 (wide, also writes the rounded f32 copy), cos in f32 (narrow)
    assert [bool(s.get("wide")) for s in chains].count(True) >= 1 and [bool(s.get("wide")) for s in chains].count(False) >= 2, p
    assert not bool(chains[0].get("wide")) and not bool(chains[-1].get("wide"))


def run64(rx, client, text, ins):
    f = rx.compile(text, client)
    out = f(*[rx.to_rarray(np.ascontiguousarray(np.asarray(a).T), client) for a in ins])
    outs = out if isinstance(out, tuple) else (out,)
    return [np.asarray(o).T for o in outs]


@pytest.mark.gpu
@pytest.mark.parametrize("case", F64_CASES, ids=[c["name"] for c in F64_CASES])
def test_f64_reference_fixtures_through_the_engine(rx, ref, client, case):
    ins = [np.array(s["data"], dtype=np.float64).reshape(s["dims"]) for s in case["inputs"]]
    got = run64(rx, client, case["module"], ins)
    for g, e in zip(got, case["expected"]):
        want = np.array(e["data"], dtype=np.float64).reshape(e["dims"])
        assert g.dtype == np.float64 and list(g.shape) == e["dims"]
        if float(case["rtol"]) == 0.0:
            assert np.array_equal(g, want)
        else:
            np.testing.assert_allclose(g, want, rtol=max(float(case["rtol"]), 1e-12))


@pytest.mark.gpu
def test_f64_elementwise_chain_matches_the_oracle(rx, ref, client):
    t, tp = "tensor<37x53xf64>", "tensor<37x53xi1>"
    text = f"""module {{
  func.func @main(%arg0: {t}, %arg1: {t}) -> ({t}, tensor<37x53xf32>, tensor<37x53xi32>) {{
    %c = stablehlo.constant dense<2.500000e-01> : {t}
    %z = stablehlo.constant dense<0.000000e+00> : {t}
    %0 = stablehlo.exponential %arg0 : {t}
    %1 = stablehlo.tanh %arg1 : {t}
    %2 = stablehlo.multiply %0, %1 : {t}
    %3 = stablehlo.add %2, %c : {t}
    %4 = stablehlo.compare GT, %3, %z : ({t}, {t}) -> {tp}
    %5 = stablehlo.sqrt %3 : {t}
    %6 = stablehlo.negate %3 : {t}
    %7 = stablehlo.select %4, %5, %6 : {tp}, {t}
    %8 = stablehlo.divide %7, %arg1 : {t}
    %9 = stablehlo.convert %8 : ({t}) -> tensor<37x53xf32>
    %10 = stablehlo.floor %8 : {t}
    %11 = stablehlo.convert %10 : ({t}) -> tensor<37x53xi32>
    return %8, %9, %11 : {t}, tensor<37x53xf32>, tensor<37x53xi32>
  }}
}}
"""
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((37, 53)), rng.standard_normal((37, 53)) + 3.0
    g = run64(rx, client, text, [a, b])
    w = ref.run_module(text, [a, b])
    np.testing.assert_allclose(g[0], w[0], rtol=1e-14)
    assert g[1].dtype == np.float32 and np.array_equal(g[1], g[0].astype(np.float32))   # rounded once from the f64 value
    assert np.array_equal(g[2], w[2])


@pytest.mark.gpu
@pytest.mark.parametrize("dims", [[0], [1], [2], [0, 1], [1, 2], [0, 2], [0, 1, 2]])
@pytest.mark.parametrize("kind", ["add", "maximum"])
def test_f64_reductions_over_every_dim_subset(rx, ref, client, dims, kind):
    shape = (12, 30, 17)
    keep = [s for d, s in enumerate(shape) if d not in dims]
    t = "tensor<12x30x17xf64>"
    tr = "tensor<" + "".join(f"{k}x" for k in keep) + "f64>"
    init = "0.000000e+00" if kind == "add" else "0xFFF0000000000000"
    text = f"""module {{
  func.func @main(%arg0: {t}) -> {tr} {{
    %cst = stablehlo.constant dense<{init}> : tensor<f64>
    %0 = stablehlo.cosine %arg0 : {t}
    %1 = stablehlo.reduce(%0 init: %cst) applies stablehlo.{kind} across dimensions = {dims} : ({t}, tensor<f64>) -> {tr}
    return %1 : {tr}
  }}
}}
"""
    x = np.random.default_rng(3).standard_normal(shape)
    (got,) = run64(rx, client, text, [x])
    want = ref.run_module(text, [x])[0]
    np.testing.assert_allclose(got, want, rtol=1e-13, atol=1e-13)


@pytest.mark.gpu
def test_f64_dot_general_and_scan(rx, ref, client):
    ta, tb, tc = "tensor<40x24xf64>", "tensor<24x31xf64>", "tensor<40x31xf64>"
    text = f"""module {{
  func.func @main(%arg0: {ta}, %arg1: {tb}) -> {tc} {{
    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : ({ta}, {tb}) -> {tc}
    return %0 : {tc}
  }}
}}
"""
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal((40, 24)), rng.standard_normal((24, 31))
    (got,) = run64(rx, client, text, [a, b])
    np.testing.assert_allclose(got, a @ b, rtol=1e-13, atol=1e-13)
