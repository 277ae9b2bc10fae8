"""Randomly generated slice-and-add window updates in counted loops: random tap sets (up to radius 2), weights, window
positions and sizes, array sizes with and without a 16-byte row pitch (TMA-staged kernel, one-launch loop, or the
strided map kernel), swapped and unswapped loop-carried arrays.  Every variant must reproduce the numpy oracle bit
for bit: the adds are evaluated in the traced order and nothing is contracted into an FMA."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()


def gen_case(seed):
    rng = np.random.default_rng(7000 + seed)
    rows = int(rng.choice([12, 33, 64, 130, 257]))
    cols = int(rng.choice([16, 36, 64, 129, 260, 516]))
    rad = int(rng.integers(1, 3))
    r0, c0 = int(rng.integers(rad, rad + 3)), int(rng.integers(rad, rad + 3))
    R = rows - r0 - int(rng.integers(rad, rad + 3))
    C = cols - c0 - int(rng.integers(rad, rad + 3))
    steps = int(rng.integers(1, 6))
    swap = bool(rng.integers(0, 2))
    t, ti = f"tensor<{rows}x{cols}xf32>", f"tensor<{R}x{C}xf32>"
    ntaps = int(rng.integers(2, 8))
    taps = []
    while len(taps) < ntaps:
        d = (int(rng.integers(-rad, rad + 1)), int(rng.integers(-rad, rad + 1)))
        if d not in taps:
            taps.append(d)
    if seed % 3 == 0:  # the 5-point cross in the order the fast path recognises
        taps = [(0, 0), (0, -1), (0, 1), (-1, 0), (1, 0)]
    lines = []
    for k, (dy, dx) in enumerate(taps):
        lines.append(f"      %s{k} = stablehlo.slice %iterArg_0 [{r0 + dy}:{r0 + dy + R}, {c0 + dx}:{c0 + dx + C}] : ({t}) -> {ti}")
    acc = "%s0"
    for k in range(1, len(taps)):
        op = "add" if seed % 3 == 0 or rng.random() < 0.7 else "subtract"
        lines.append(f"      %a{k} = stablehlo.{op} {acc}, %s{k} : {ti}")
        acc = f"%a{k}"
    w = float(np.float32(rng.choice([0.2, 0.125, 1.0 / 3.0, 0.37])))
    lines.append(f"      %u = stablehlo.multiply %cst, {acc} : {ti}")
    lines.append(f"      %nb = stablehlo.dynamic_update_slice %iterArg_1, %u, %c_r, %c_c : ({t}, {ti}, tensor<i32>, tensor<i32>) -> {t}")
    body = "\n".join(lines)
    yields = "%1, %nb, %iterArg_0" if swap else "%1, %iterArg_0, %nb"
    text = f"""module @reactant_stencil attributes {{mhlo.num_partitions = 1 : i64, mhlo.num_replicas = 1 : i64}} {{
  func.func @main(%arg0: {t} {{tf.aliasing_output = 0 : i32}}, %arg1: {t} {{tf.aliasing_output = 1 : i32}}) -> ({t}, {t}) {{
    %c = stablehlo.constant dense<0> : tensor<i64>
    %c_0 = stablehlo.constant dense<{steps}> : tensor<i64>
    %c_2 = stablehlo.constant dense<1> : tensor<i64>
    %c_r = stablehlo.constant dense<{r0}> : tensor<i32>
    %c_c = stablehlo.constant dense<{c0}> : tensor<i32>
    %cst = stablehlo.constant dense<{w!r}> : {ti}
    %0:3 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0, %iterArg_1 = %arg1) : tensor<i64>, {t}, {t}
     cond {{
      %1 = stablehlo.compare  LT, %iterArg, %c_0 : (tensor<i64>, tensor<i64>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    }} do {{
      %1 = stablehlo.add %iterArg, %c_2 : tensor<i64>
{body}
      stablehlo.return {yields} : tensor<i64>, {t}, {t}
    }}
    return %0#1, %0#2 : {t}, {t}
  }}
}}
"""
    a = rng.random((rows, cols), dtype=np.float32)
    b = rng.random((rows, cols), dtype=np.float32)
    return text, [a, b]


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("RX_FUZZ_FIRST", "0")), int(os.environ.get("RX_FUZZ_FIRST", "0")) + int(os.environ.get("RX_FUZZ_CASES", "60"))))
def test_random_window_updates_in_loops(seed):
    oracle, _ = entry.load_oracle()
    text, inputs = gen_case(seed)
    want = oracle.run_module(text, inputs)
    f = rx.compile(text)
    r = f(*[rx.to_rarray(np.ascontiguousarray(a.T)) for a in inputs])
    got = [np.ascontiguousarray(np.asarray(t).T) for t in r]
    for g, w in zip(got, want):
        assert np.array_equal(g, np.asarray(w, dtype=np.float32)), text
