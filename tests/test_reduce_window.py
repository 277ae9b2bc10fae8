"""stablehlo.reduce_window beyond scans: pooling windows with strides, padding and window dilations
(ext/ReactantNNlibExt/Implementations.jl pooling, src/TracedRArray.jl:981-1047).  The planner turns them into one
strided view of the (padded) operand per window position, combined by an ordinary fused chain.  CPU: the oracle
against direct numpy pooling, and the plans.  GPU: the engine against the oracle -- bit-exact for max / min and
integer sums, within the fp32 reduction tolerance for float sums (the order of the additions is not specified)."""
import numpy as np
import pytest


def window_module(shape, win, strides, pad, dil, kind, et="f32"):
    rank = len(shape)
    span = [(w - 1) * d + 1 for w, d in zip(win, dil)]
    out = [(s + lo + hi - sp) // st + 1 for s, (lo, hi), sp, st in zip(shape, pad, span, strides)]
    tin = "tensor<" + "x".join(map(str, shape)) + f"x{et}>"
    tout = "tensor<" + "x".join(map(str, out)) + f"x{et}>"
    ts = f"tensor<{et}>"
    if et == "f32":
        init = {"add": "0.000000e+00", "maximum": "0xFF800000", "minimum": "0x7F800000", "multiply": "1.000000e+00"}[kind]
    else:
        init = {"add": "0", "maximum": str(-2**31), "minimum": str(2**31 - 1), "multiply": "1"}[kind]
    padtxt = "[" + ", ".join(f"[{lo}, {hi}]" for lo, hi in pad) + "]"
    arr = lambda v: "array<i64: " + ", ".join(map(str, v)) + ">"
    text = f"""module {{
  func.func @main(%arg0: {tin}) -> {tout} {{
    %c = stablehlo.constant dense<{init}> : {ts}
    %0 = "stablehlo.reduce_window"(%arg0, %c) <{{padding = dense<{padtxt}> : tensor<{rank}x2xi64>, window_dilations = {arr(dil)}, window_dimensions = {arr(win)}, window_strides = {arr(strides)}}}> ({{
    ^bb0(%a: {ts}, %b: {ts}):
      %m = stablehlo.{kind} %a, %b : {ts}
      stablehlo.return %m : {ts}
    }}) : ({tin}, {ts}) -> {tout}
    return %0 : {tout}
  }}
}}
"""
    return text, out


CASES = [
    # shape, window, strides, padding, window dilations, combiner
    ((64, 96), (2, 2), (2, 2), ((0, 0), (0, 0)), (1, 1), "maximum"),        # 2 x 2 max pooling
    ((64, 96), (3, 3), (2, 2), ((1, 1), (1, 1)), (1, 1), "maximum"),        # 3 x 3, stride 2, same padding: 9 positions -> two chains
    ((33, 70), (3, 3), (1, 1), ((1, 1), (1, 1)), (1, 1), "add"),            # 3 x 3 box sum
    ((4, 6, 30, 20), (1, 1, 2, 2), (1, 1, 2, 2), ((0, 0),) * 4, (1, 1, 1, 1), "add"),   # NCHW mean-pool numerator
    ((40, 50), (2, 3), (1, 2), ((0, 1), (2, 0)), (2, 1), "minimum"),        # ragged: dilation, asymmetric padding
    ((5, 1000), (1, 7), (1, 3), ((0, 0), (3, 3)), (1, 1), "maximum"),       # 1-D window along the contiguous dim
]


def test_oracle_agrees_with_direct_pooling(ref):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((6, 8)).astype(np.float32)
    text, _ = window_module((6, 8), (2, 2), (2, 2), ((0, 0), (0, 0)), (1, 1), "maximum")
    assert np.array_equal(ref.run_module(text, [x])[0], x.reshape(3, 2, 4, 2).max(axis=(1, 3)))
    text, _ = window_module((6, 8), (3, 3), (1, 1), ((1, 1), (1, 1)), (1, 1), "add")
    p = np.pad(x.astype(np.float64), 1)
    want = sum(p[i:i + 6, j:j + 8] for i in range(3) for j in range(3)).astype(np.float32)
    np.testing.assert_allclose(ref.run_module(text, [x])[0], want, rtol=1e-6)


def test_windows_plan_as_fused_chains_over_strided_views(rx):
    kinds = lambda p: [s["kind"] for s in p["steps"]]
    text, _ = window_module(*CASES[0])
    assert kinds(rx.plan_describe(text)) == ["map"]                       # four views, one chain
    text, _ = window_module(*CASES[1])
    k = kinds(rx.plan_describe(text))
    assert k == ["map", "map", "map", "map"], k                            # padding fill + interior, partial after six positions, rest
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(window_module((64, 64), (9, 9), (1, 1), ((0, 0), (0, 0)), (1, 1), "add")[0])
    assert e.value.code == 2 and "more than 64" in str(e.value)
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(window_module((64, 64), (2, 2), (2, 2), ((0, 0), (0, 0)), (1, 1), "add")[0].replace("window_dilations", "base_dilations = array<i64: 2, 1>, window_dilations"))
    assert e.value.code == 2 and "base_dilations" in str(e.value)


@pytest.mark.gpu
@pytest.mark.parametrize("case", range(len(CASES)))
def test_window_reductions_match_the_oracle(rx, ref, client, case):
    shape, win, strides, pad, dil, kind = CASES[case]
    text, out = window_module(shape, win, strides, pad, dil, kind)
    rng = np.random.default_rng(case)
    x = rng.standard_normal(shape).astype(np.float32)
    got = np.asarray(rx.compile(text, client)(rx.to_rarray(np.ascontiguousarray(x.T), client))).T
    want = ref.run_module(text, [x])[0]
    assert got.shape == tuple(out)
    if kind in ("maximum", "minimum"):
        assert np.array_equal(got, want)
    else:
        np.testing.assert_allclose(got, want, rtol=0, atol=1e-5 * np.sqrt(float(np.prod(win))) * np.abs(x).max() * np.prod(win))


@pytest.mark.gpu
def test_integer_window_sum_is_exact(rx, ref, client):
    text, _ = window_module((50, 60), (2, 3), (2, 3), ((0, 0), (0, 0)), (1, 1), "add", et="i32")
    x = np.random.default_rng(1).integers(-1000, 1000, (50, 60)).astype(np.int32)
    got = np.asarray(rx.compile(text, client)(rx.to_rarray(np.ascontiguousarray(x.T), client))).T
    assert np.array_equal(got, ref.run_module(text, [x])[0])
