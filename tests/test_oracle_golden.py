"""The CPU oracle against the known-answer fixtures of Reactant's own tests
(tests/golden/reactant_fixtures.json) and the C kernels against the numpy
interpreter.  No GPU."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reactant_fixtures.json")) as f:
    CASES = json.load(f)["cases"]

NP = {"f64": np.float64, "f32": np.float32, "i32": np.int32, "i1": np.bool_}


def case_inputs(case, ref):
    mod = ref.parse_module(case["module"])
    args = mod["funcs"]["main"].args
    out = []
    for (name, (shape, et)), spec in zip(args, case["inputs"]):
        out.append(np.array(spec["data"], dtype=NP[et]).reshape(spec["dims"]))
    return out


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_fixture(case, ref):
    got = ref.run_module(case["module"], case_inputs(case, ref))
    assert len(got) == len(case["expected"])
    for g, e in zip(got, case["expected"]):
        want = np.array(e["data"], dtype=np.float64).reshape(e["dims"])
        assert list(g.shape) == e["dims"]
        if case["rtol"] == 0.0:
            assert np.array_equal(g, want.astype(g.dtype)), case["name"]  # exact in the element type
        else:
            np.testing.assert_allclose(g.astype(np.float64), want, rtol=case["rtol"], atol=0)


def test_c_sinsum_matches_interpreter(ref, cpu):
    import __graft_entry__ as entry
    rx_programs = entry._load_file("rx_programs_only", os.path.join(entry.PKG_DIR, "programs.py"))
    rng = np.random.default_rng(1)
    for n in (1, 3, 127, 4097, (1 << 18) + 1):
        x = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
        y = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
        want = float(ref.run_module(rx_programs.sinsum_add(n), [x, y])[0])
        got = cpu.sinsum_add(x, y)
        scale = float(np.sqrt(np.sum((np.sin(x.astype(np.float64)) + y) ** 2))) + 1e-30
        assert abs(got - want) <= ref.reduction_tolerance(n) * max(abs(want), scale)


def test_c_logsumexp_matches_interpreter(ref, cpu):
    import __graft_entry__ as entry
    P = entry._load_file("rx_programs_only", os.path.join(entry.PKG_DIR, "programs.py"))
    rng = np.random.default_rng(3)
    for rows, cols in ((1, 1), (7, 3), (1000, 17), (4096, 8)):
        x = rng.standard_normal((cols, rows)).astype(np.float32)  # boundary layout
        for raw in (False, True):
            want = ref.run_module(P.logsumexp_dims1(rows, cols, raw=raw), [x])[0].reshape(-1)
            np.testing.assert_allclose(cpu.logsumexp_dims1(x), want, rtol=ref.reduction_tolerance(rows))


def test_c_jacobi_matches_interpreter_bit_exact(ref, cpu):
    import __graft_entry__ as entry
    P = entry._load_file("rx_programs_only", os.path.join(entry.PKG_DIR, "programs.py"))
    rng = np.random.default_rng(4)
    for n, steps in ((3, 1), (8, 2), (33, 5)):
        a = rng.random((n, n), dtype=np.float32)
        b = rng.random((n, n), dtype=np.float32)
        for form in ("dus", "pad"):
            wa, wb = ref.run_module(P.jacobi2d(n, steps, form=form), [a, b])
            ga, gb = cpu.jacobi2d(a, b, steps)
            assert np.array_equal(ga, wa) and np.array_equal(gb, wb), (n, steps, form)


def test_bf16_rounding_is_nearest_even(ref):
    x = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.0e38, 1e-40], dtype=np.float32)
    r = ref.round_to_bf16(x)
    # 1.00390625 = 1 + 2^-8 is a tie between 1.0 and 1.0078125 -> even mantissa (1.0)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625) and r[3] == -1.0
    import ml_dtypes
    assert np.array_equal(r, x.astype(ml_dtypes.bfloat16).astype(np.float32))
