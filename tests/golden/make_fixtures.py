"""Generates tests/golden/reactant_fixtures.json.

Each case restates one known-answer test of Reactant.jl's own suite for the hot
path: the closed-form input of the test (Reactant.TestUtils.construct_test_array,
src/TestUtils.jl:9-23), the StableHLO module the traced Julia function lowers to
(written by hand from the op emitters, in the reversed-dims boundary layout),
and the value native Julia computes for it.  The reference compares against
native Julia, not against stored numbers, so the expected values here are
recomputed from the closed forms with exact rational / math-library arithmetic
in pure Python (no numpy, no oracle code), which is what pins the oracle.

Run: python tests/golden/make_fixtures.py   (rewrites the JSON next to it)
"""
from __future__ import annotations

import json
import math
import os
from fractions import Fraction

HERE = os.path.dirname(os.path.abspath(__file__))


def t(shape, et):
    return "tensor<" + "".join(f"{d}x" for d in shape) + et + ">"


def wrap(args, results, body):
    a = ", ".join(f"%arg{i}: {ty}" for i, ty in enumerate(args))
    r = ", ".join(results)
    return f"module {{\n  func.func @main({a}) -> ({r}) {{\n{body}\n  }}\n}}\n"


def cta(*dims):
    """construct_test_array(Float, dims...) as a flat column-major list of Fractions."""
    n = math.prod(dims)
    return [Fraction(k, n) for k in range(1, n + 1)]


def col_major_to_xla(flat, dims):
    """Column-major Julia data == row-major data of the reversed dims: bytes unchanged."""
    return flat


def idx_cm(dims, *ix):
    """0-based column-major linear index."""
    lin, mul = 0, 1
    for d, i in zip(dims, ix):
        lin += i * mul
        mul *= d
    return lin


cases = []


def add(name, source, module, inputs, expected, et, tol):
    cases.append({"name": name, "reference_test": source, "module": module, "inputs": inputs,
                  "expected": expected, "element_type": et, "rtol": tol})


for et in ("f64", "f32"):
    tol = 1e-12 if et == "f64" else 2e-6
    # ---- test/core/map_reduction.jl:8-19  "2D sum": sum(construct_test_array(Float64, 2, 10)) ----
    x = cta(2, 10)
    add(f"sum_2d_{et}", "test/core/map_reduction.jl:8-19",
        wrap([t([10, 2], et)], [t([], et)],
             f"    %cst = stablehlo.constant dense<0.000000e+00> : {t([], et)}\n"
             f"    %0 = stablehlo.reduce(%arg0 init: %cst) applies stablehlo.add across dimensions = [0, 1] : ({t([10, 2], et)}, {t([], et)}) -> {t([], et)}\n"
             f"    return %0 : {t([], et)}"),
        [{"dims": [10, 2], "data": [float(v) for v in x]}],
        [{"dims": [], "data": [float(sum(x))]}], et, tol)

    # ---- :21-32 "Basic reduce max": reduce(max, x; dims=1, init=-Inf) on 2x10 -> 1x10 ----
    neg_inf = "0xFFF0000000000000" if et == "f64" else "0xFF800000"
    mx = [max(x[idx_cm((2, 10), 0, j)], x[idx_cm((2, 10), 1, j)]) for j in range(10)]
    add(f"reduce_max_dims1_{et}", "test/core/map_reduction.jl:21-32",
        wrap([t([10, 2], et)], [t([10, 1], et)],
             f"    %cst = stablehlo.constant dense<{neg_inf}> : {t([], et)}\n"
             f"    %0 = stablehlo.reduce(%arg0 init: %cst) applies stablehlo.maximum across dimensions = [1] : ({t([10, 2], et)}, {t([], et)}) -> {t([10], et)}\n"
             f"    %1 = stablehlo.reshape %0 : ({t([10], et)}) -> {t([10, 1], et)}\n"
             f"    return %1 : {t([10, 1], et)}"),
        [{"dims": [10, 2], "data": [float(v) for v in x]}],
        [{"dims": [10, 1], "data": [float(v) for v in mx]}], et, tol)

    # ---- :60-73 "Basic softmax": x .- reduce(max, x; dims=1, init=-Inf) ----
    sm = [float(x[idx_cm((2, 10), i, j)] - mx[j]) for j in range(10) for i in range(2)]
    add(f"softmax_core_{et}", "test/core/map_reduction.jl:60-73",
        wrap([t([10, 2], et)], [t([10, 2], et)],
             f"    %cst = stablehlo.constant dense<{neg_inf}> : {t([], et)}\n"
             f"    %0 = stablehlo.reduce(%arg0 init: %cst) applies stablehlo.maximum across dimensions = [1] : ({t([10, 2], et)}, {t([], et)}) -> {t([10], et)}\n"
             f"    %1 = stablehlo.broadcast_in_dim %0, dims = [0] : ({t([10], et)}) -> {t([10, 2], et)}\n"
             f"    %2 = stablehlo.subtract %arg0, %1 : {t([10, 2], et)}\n"
             f"    return %2 : {t([10, 2], et)}"),
        [{"dims": [10, 2], "data": [float(v) for v in x]}],
        [{"dims": [10, 2], "data": sm}], et, tol)

    # ---- :75-86 sum(x .* x') on construct_test_array(Float64, 4, 4) ----
    x4 = cta(4, 4)
    s = sum(x4[idx_cm((4, 4), i, j)] * x4[idx_cm((4, 4), j, i)] for i in range(4) for j in range(4))
    add(f"sum_x_xt_{et}", "test/core/map_reduction.jl:75-86",
        wrap([t([4, 4], et)], [t([], et)],
             f"    %cst = stablehlo.constant dense<0.000000e+00> : {t([], et)}\n"
             f"    %0 = stablehlo.transpose %arg0, dims = [1, 0] : ({t([4, 4], et)}) -> {t([4, 4], et)}\n"
             f"    %1 = stablehlo.multiply %arg0, %0 : {t([4, 4], et)}\n"
             f"    %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [0, 1] : ({t([4, 4], et)}, {t([], et)}) -> {t([], et)}\n"
             f"    return %2 : {t([], et)}"),
        [{"dims": [4, 4], "data": [float(v) for v in x4]}],
        [{"dims": [], "data": [float(s)]}], et, tol)

    # ---- :147-161 "mapreducedim!": x = reshape(1:64, 2,4,8)./64 ; sum!(y(1,1,8), x) and sum(abs2) to (2,1,1) ----
    x3 = [Fraction(k, 64) for k in range(1, 65)]
    dims3 = (2, 4, 8)
    f1 = [float(sum(x3[idx_cm(dims3, i, j, k)] for i in range(2) for j in range(4))) for k in range(8)]
    add(f"sum_dims12_{et}", "test/core/map_reduction.jl:147-161 (fntest1, sum(x; dims=1:2))",
        wrap([t([8, 4, 2], et)], [t([8, 1, 1], et)],
             f"    %cst = stablehlo.constant dense<0.000000e+00> : {t([], et)}\n"
             f"    %0 = stablehlo.reduce(%arg0 init: %cst) applies stablehlo.add across dimensions = [1, 2] : ({t([8, 4, 2], et)}, {t([], et)}) -> {t([8], et)}\n"
             f"    %1 = stablehlo.reshape %0 : ({t([8], et)}) -> {t([8, 1, 1], et)}\n"
             f"    return %1 : {t([8, 1, 1], et)}"),
        [{"dims": [8, 4, 2], "data": [float(v) for v in x3]}],
        [{"dims": [8, 1, 1], "data": f1}], et, tol)
    f2 = [float(sum(x3[idx_cm(dims3, i, j, k)] for j in range(4))) for k in range(8) for i in range(2)]
    add(f"sum_dim2_{et}", "test/core/map_reduction.jl:147-161 (fntest2)",
        wrap([t([8, 4, 2], et)], [t([8, 1, 2], et)],
             f"    %cst = stablehlo.constant dense<0.000000e+00> : {t([], et)}\n"
             f"    %0 = stablehlo.reduce(%arg0 init: %cst) applies stablehlo.add across dimensions = [1] : ({t([8, 4, 2], et)}, {t([], et)}) -> {t([8, 2], et)}\n"
             f"    %1 = stablehlo.reshape %0 : ({t([8, 2], et)}) -> {t([8, 1, 2], et)}\n"
             f"    return %1 : {t([8, 1, 2], et)}"),
        [{"dims": [8, 4, 2], "data": [float(v) for v in x3]}],
        [{"dims": [8, 1, 2], "data": f2}], et, tol)
    f3 = [float(sum(x3[idx_cm(dims3, i, j, k)] ** 2 for j in range(4) for k in range(8))) for i in range(2)]
    add(f"sum_abs2_dims23_{et}", "test/core/map_reduction.jl:147-161 (fntest3)",
        wrap([t([8, 4, 2], et)], [t([1, 1, 2], et)],
             f"    %cst = stablehlo.constant dense<0.000000e+00> : {t([], et)}\n"
             f"    %0 = stablehlo.multiply %arg0, %arg0 : {t([8, 4, 2], et)}\n"
             f"    %1 = stablehlo.reduce(%0 init: %cst) applies stablehlo.add across dimensions = [0, 1] : ({t([8, 4, 2], et)}, {t([], et)}) -> {t([2], et)}\n"
             f"    %2 = stablehlo.reshape %1 : ({t([2], et)}) -> {t([1, 1, 2], et)}\n"
             f"    return %2 : {t([1, 1, 2], et)}"),
        [{"dims": [8, 4, 2], "data": [float(v) for v in x3]}],
        [{"dims": [1, 1, 2], "data": f3}], et, tol)

    # ---- test/core/indexing.jl:3-29 update_on_copy: y = x[1:2, 2:4, :]; y[1:1, 1:1, :] = ones(1,1,3) ----
    xi = cta(2, 4, 3)
    y = {}
    for i in range(2):
        for j in range(3):
            for k in range(3):
                y[(i, j, k)] = xi[idx_cm((2, 4, 3), i, j + 1, k)]
    for k in range(3):
        y[(0, 0, k)] = Fraction(1)
    yflat = [float(y[(i, j, k)]) for k in range(3) for j in range(3) for i in range(2)]
    one = "1.000000e+00"
    add(f"slice_update_{et}", "test/core/indexing.jl:3-29",
        wrap([t([3, 4, 2], et)], [t([3, 3, 2], et)],
             f"    %c = stablehlo.constant dense<0> : tensor<i32>\n"
             f"    %ones = stablehlo.constant dense<{one}> : {t([3, 1, 1], et)}\n"
             f"    %0 = stablehlo.slice %arg0 [0:3, 1:4, 0:2] : ({t([3, 4, 2], et)}) -> {t([3, 3, 2], et)}\n"
             f"    %1 = stablehlo.dynamic_update_slice %0, %ones, %c, %c, %c : ({t([3, 3, 2], et)}, {t([3, 1, 1], et)}, tensor<i32>, tensor<i32>, tensor<i32>) -> {t([3, 3, 2], et)}\n"
             f"    return %1 : {t([3, 3, 2], et)}"),
        [{"dims": [3, 4, 2], "data": [float(v) for v in xi]}],
        [{"dims": [3, 3, 2], "data": yflat}], et, 0.0)

    # ---- test/core/compile.jl:350-355 "matmul": ones(50,70) * ones(70,30) == 70 everywhere ----
    add(f"matmul_ones_{et}", "test/core/compile.jl:350-355",
        wrap([t([70, 50], et), t([30, 70], et)], [t([30, 50], et)],
             f"    %0 = stablehlo.dot_general %arg1, %arg0, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : ({t([30, 70], et)}, {t([70, 50], et)}) -> {t([30, 50], et)}\n"
             f"    return %0 : {t([30, 50], et)}"),
        [{"dims": [70, 50], "data": [1.0] * 3500}, {"dims": [30, 70], "data": [1.0] * 2100}],
        [{"dims": [30, 50], "data": [70.0] * 1500}], et, 0.0)

# ---- :42-58 "Basic mapreduce": sum(exp, construct_test_array(Float32, 10)) ----
import struct


def f32(v):
    return struct.unpack("f", struct.pack("f", v))[0]


x10 = [f32(k / 10) for k in range(1, 11)]
add("sum_exp_f32", "test/core/map_reduction.jl:42-58",
    wrap([t([10], "f32")], [t([], "f32")],
         "    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
         "    %0 = stablehlo.exponential %arg0 : tensor<10xf32>\n"
         "    %1 = stablehlo.reduce(%0 init: %cst) applies stablehlo.add across dimensions = [0] : (tensor<10xf32>, tensor<f32>) -> tensor<f32>\n"
         "    return %1 : tensor<f32>"),
    [{"dims": [10], "data": x10}], [{"dims": [], "data": [math.fsum(math.exp(v) for v in x10)]}], "f32", 2e-6)

# ---- test/nn/nnlib.jl:94-101 logsumexp(collect(Float32, 1:16)) ----
x16 = [float(k) for k in range(1, 17)]
lse16 = 16.0 + math.log(math.fsum(math.exp(v - 16.0) for v in x16))
add("logsumexp_1to16_f32", "test/nn/nnlib.jl:94-101",
    wrap([t([16], "f32")], [t([], "f32")],
         "    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
         "    %cst_0 = stablehlo.constant dense<0xFF800000> : tensor<f32>\n"
         "    %0 = stablehlo.reduce(%arg0 init: %cst_0) applies stablehlo.maximum across dimensions = [0] : (tensor<16xf32>, tensor<f32>) -> tensor<f32>\n"
         "    %1 = stablehlo.broadcast_in_dim %0, dims = [] : (tensor<f32>) -> tensor<16xf32>\n"
         "    %2 = stablehlo.subtract %arg0, %1 : tensor<16xf32>\n"
         "    %3 = stablehlo.exponential %2 : tensor<16xf32>\n"
         "    %4 = stablehlo.reduce(%3 init: %cst) applies stablehlo.add across dimensions = [0] : (tensor<16xf32>, tensor<f32>) -> tensor<f32>\n"
         "    %5 = stablehlo.log %4 : tensor<f32>\n"
         "    %6 = stablehlo.add %0, %5 : tensor<f32>\n"
         "    return %6 : tensor<f32>"),
    [{"dims": [16], "data": x16}], [{"dims": [], "data": [lse16]}], "f32", 2e-6)

# ---- test/integration/log_exp_functions.jl:315-338 logsumexp([1 2; 3 4]; dims=1 / dims=2) ----
M = {(0, 0): 1.0, (0, 1): 2.0, (1, 0): 3.0, (1, 1): 4.0}
flat = [M[(i, j)] for j in range(2) for i in range(2)]  # column-major
d1 = [max(M[(0, j)], M[(1, j)]) + math.log(sum(math.exp(M[(i, j)] - max(M[(0, j)], M[(1, j)])) for i in range(2))) for j in range(2)]
d2 = [max(M[(i, 0)], M[(i, 1)]) + math.log(sum(math.exp(M[(i, j)] - max(M[(i, 0)], M[(i, 1)])) for j in range(2))) for i in range(2)]
for name, dim, exp_, oshape in (("dims1", 1, d1, [2, 1]), ("dims2", 0, d2, [1, 2])):
    red = [2]
    bdims = "[0]" if dim == 1 else "[1]"
    add(f"logsumexp_2x2_{name}_f32", "test/integration/log_exp_functions.jl:315-338",
        wrap([t([2, 2], "f32")], [t(oshape, "f32")],
             "    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
             "    %cst_0 = stablehlo.constant dense<0xFF800000> : tensor<f32>\n"
             f"    %0 = stablehlo.reduce(%arg0 init: %cst_0) applies stablehlo.maximum across dimensions = [{dim}] : (tensor<2x2xf32>, tensor<f32>) -> tensor<2xf32>\n"
             f"    %1 = stablehlo.broadcast_in_dim %0, dims = {bdims} : (tensor<2xf32>) -> tensor<2x2xf32>\n"
             "    %2 = stablehlo.subtract %arg0, %1 : tensor<2x2xf32>\n"
             "    %3 = stablehlo.exponential %2 : tensor<2x2xf32>\n"
             f"    %4 = stablehlo.reduce(%3 init: %cst) applies stablehlo.add across dimensions = [{dim}] : (tensor<2x2xf32>, tensor<f32>) -> tensor<2xf32>\n"
             "    %5 = stablehlo.log %4 : tensor<2xf32>\n"
             "    %6 = stablehlo.add %0, %5 : tensor<2xf32>\n"
             f"    %7 = stablehlo.reshape %6 : (tensor<2xf32>) -> {t(oshape, 'f32')}\n"
             f"    return %7 : {t(oshape, 'f32')}"),
        [{"dims": [2, 2], "data": flat}], [{"dims": oshape, "data": exp_}], "f32", 2e-6)

# ---- test/core/indexing.jl:140-157 strided: x = reshape(collect(1:24), 4, 6); x[1:2:4, 3:2:6] (Int32 here) ----
xs = list(range(1, 25))
sel = [xs[idx_cm((4, 6), i, j)] for j in (2, 4) for i in (0, 2)]
add("strided_slice_i32", "test/core/indexing.jl:140-157",
    wrap([t([6, 4], "i32")], [t([2, 2], "i32")],
         "    %0 = stablehlo.slice %arg0 [2:5:2, 0:3:2] : (tensor<6x4xi32>) -> tensor<2x2xi32>\n"
         "    return %0 : tensor<2x2xi32>"),
    [{"dims": [6, 4], "data": xs}], [{"dims": [2, 2], "data": sel}], "i32", 0.0)

# ---- test/core/map_reduction.jl:88-98 "reduce integers": sum(Int 1:100) (Int32 here) and count of odd ----
add("sum_int_1to100_i32", "test/core/map_reduction.jl:88-98",
    wrap([t([100], "i32")], [t([], "i32")],
         "    %c = stablehlo.constant dense<0> : tensor<i32>\n"
         "    %0 = stablehlo.reduce(%arg0 init: %c) applies stablehlo.add across dimensions = [0] : (tensor<100xi32>, tensor<i32>) -> tensor<i32>\n"
         "    return %0 : tensor<i32>"),
    [{"dims": [100], "data": list(range(1, 101))}], [{"dims": [], "data": [5050]}], "i32", 0.0)
add("count_odd_bool_i32", "test/core/map_reduction.jl:88-98 (sum of Bool widens to Int)",
    wrap([t([100], "i1")], [t([], "i32")],
         "    %c = stablehlo.constant dense<0> : tensor<i32>\n"
         "    %0 = stablehlo.convert %arg0 : (tensor<100xi1>) -> tensor<100xi32>\n"
         "    %1 = stablehlo.reduce(%0 init: %c) applies stablehlo.add across dimensions = [0] : (tensor<100xi32>, tensor<i32>) -> tensor<i32>\n"
         "    return %1 : tensor<i32>"),
    [{"dims": [100], "data": [k % 2 for k in range(1, 101)]}], [{"dims": [], "data": [50]}], "i32", 0.0)

# ---- test/core/sharding/sharding.jl:26-63: sum over a sharded vector equals the unsharded sum ----
xsh = [Fraction(k, 768) for k in range(1, 769)]
add("sharded_sum_768_f32", "test/core/sharding/sharding.jl:26-63 (collect(1:768)/768, full sum, 8 devices)",
    "module attributes {mhlo.num_partitions = 8 : i64, mhlo.num_replicas = 1 : i64} {\n"
    '  sdy.mesh @mesh = <["x"=8]>\n'
    '  func.func @main(%arg0: tensor<768xf32> {sdy.sharding = #sdy.sharding<@mesh, [{"x"}]>}) -> tensor<f32> {\n'
    "    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
    "    %0 = stablehlo.reduce(%arg0 init: %cst) applies stablehlo.add across dimensions = [0] : (tensor<768xf32>, tensor<f32>) -> tensor<f32>\n"
    "    return %0 : tensor<f32>\n  }\n}\n",
    [{"dims": [768], "data": [float(v) for v in xsh]}], [{"dims": [], "data": [float(sum(xsh))]}], "f32", 2e-6)

# ---- test/core/map_reduction.jl:163-200 "accumulate" / "cumsum": a = (1:10)/10; b = reshape(1:60, 3,4,5)/60, dims = 1, 2, 3 ----
# Reactant lowers cumsum to stablehlo.reduce_window over the whole dimension, padded low by its extent minus one
# (scan_impl!, src/TracedRArray.jl:1049-1107); MLIR prints that op in the generic form.
def reduce_window_module(xla_dims, xla_axis, et, kind="add", init="0.000000e+00"):
    rank = len(xla_dims)
    win = [1] * rank
    win[xla_axis] = xla_dims[xla_axis]
    pad = [[0, 0] for _ in range(rank)]
    pad[xla_axis] = [xla_dims[xla_axis] - 1, 0]
    ones = ", ".join(["1"] * rank)
    ty = t(xla_dims, et)
    pads = "[" + ", ".join(f"[{lo}, {hi}]" for lo, hi in pad) + "]"
    return wrap([ty], [ty],
                f"    %cst = stablehlo.constant dense<{init}> : {t([], et)}\n"
                f"    %0 = \"stablehlo.reduce_window\"(%arg0, %cst) <{{base_dilations = array<i64: {ones}>, padding = dense<{pads}> : tensor<{rank}x2xi64>, "
                f"window_dilations = array<i64: {ones}>, window_dimensions = array<i64: {', '.join(map(str, win))}>, window_strides = array<i64: {ones}>}}> ({{\n"
                f"    ^bb0(%arg1: {t([], et)}, %arg2: {t([], et)}):\n"
                f"      %1 = stablehlo.{kind} %arg1, %arg2 : {t([], et)}\n"
                f"      stablehlo.return %1 : {t([], et)}\n"
                f"    }}) : ({ty}, {t([], et)}) -> {ty}\n"
                f"    return %0 : {ty}")


for et in ("f64", "f32"):
    tol = 1e-12 if et == "f64" else 2e-6
    a10 = [Fraction(k, 10) for k in range(1, 11)]
    run, acc = [], Fraction(0)
    for v in a10:
        acc += v
        run.append(float(acc))
    add(f"cumsum_vector_{et}", "test/core/map_reduction.jl:163-173 (cumsum(a), a = (1:10)/10)",
        reduce_window_module([10], 0, et), [{"dims": [10], "data": [float(v) for v in a10]}], [{"dims": [10], "data": run}], et, tol)
    b60 = [Fraction(k, 60) for k in range(1, 61)]
    jd = (3, 4, 5)
    for jdim in (1, 2, 3):
        out = [None] * 60
        for i in range(3):
            for j in range(4):
                for k in range(5):
                    ix = [i, j, k]
                    acc = Fraction(0)
                    for q in range(ix[jdim - 1] + 1):
                        jx = list(ix)
                        jx[jdim - 1] = q
                        acc += b60[idx_cm(jd, *jx)]
                    out[idx_cm(jd, i, j, k)] = float(acc)
        add(f"cumsum_3d_dims{jdim}_{et}", f"test/core/map_reduction.jl:175-177 (cumsum(b; dims={jdim}), b = reshape(1:60, 3, 4, 5)/60)",
            reduce_window_module([5, 4, 3], 3 - jdim, et), [{"dims": [5, 4, 3], "data": [float(v) for v in b60]}],
            [{"dims": [5, 4, 3], "data": out}], et, tol)

# ---- test/nn/activations.jl:3-33 "Activation Functions": sumabs2(act, x) = sum(abs2, act.(x)) on
# x = construct_test_array(Float32, 10, 10) .- 0.5f0, for act in (tanh, sigmoid, gelu).  gelu is NNlib's tanh form,
# which Reactant emits as enzymexla.math_gelu {TANH} and lowers to tanh / multiply / add
# (ext/ReactantNNlibExt/Implementations.jl:12-25, src/Ops.jl:4153-4175).
import struct


def f32(v):
    return struct.unpack("f", struct.pack("f", float(v)))[0]


x_act = [f32(f32(float(Fraction(k, 100))) - 0.5) for k in range(1, 101)]
T100 = t([10, 10], "f32")


def sumabs2_module(body_lines, last):
    return wrap([T100], [t([], "f32")],
                "\n".join(body_lines) + "\n"
                f"    %sq = stablehlo.multiply {last}, {last} : {T100}\n"
                f"    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
                f"    %r = stablehlo.reduce(%sq init: %cst) applies stablehlo.add across dimensions = [0, 1] : ({T100}, tensor<f32>) -> tensor<f32>\n"
                f"    return %r : tensor<f32>")


add("sumabs2_tanh_f32", "test/nn/activations.jl:3-33 (act = tanh)",
    sumabs2_module([f"    %0 = stablehlo.tanh %arg0 : {T100}"], "%0"),
    [{"dims": [10, 10], "data": x_act}], [{"dims": [], "data": [sum(math.tanh(v) ** 2 for v in x_act)]}], "f32", 5e-6)
add("sumabs2_sigmoid_f32", "test/nn/activations.jl:3-33 (act = sigmoid)",
    sumabs2_module([f"    %0 = stablehlo.logistic %arg0 : {T100}"], "%0"),
    [{"dims": [10, 10], "data": x_act}], [{"dims": [], "data": [sum((1.0 / (1.0 + math.exp(-v))) ** 2 for v in x_act)]}], "f32", 5e-6)
c0, c1 = f32(math.sqrt(2.0 / math.pi)), f32(0.044715)
gelu_lines = [
    f"    %k0 = stablehlo.constant dense<{c0!r}> : {T100}",
    f"    %k1 = stablehlo.constant dense<{c1!r}> : {T100}",
    f"    %half = stablehlo.constant dense<5.000000e-01> : {T100}",
    f"    %one = stablehlo.constant dense<1.000000e+00> : {T100}",
    f"    %x2 = stablehlo.multiply %arg0, %arg0 : {T100}",
    f"    %x3 = stablehlo.multiply %x2, %arg0 : {T100}",
    f"    %a = stablehlo.multiply %k1, %x3 : {T100}",
    f"    %b = stablehlo.add %arg0, %a : {T100}",
    f"    %c = stablehlo.multiply %k0, %b : {T100}",
    f"    %th = stablehlo.tanh %c : {T100}",
    f"    %d = stablehlo.add %one, %th : {T100}",
    f"    %e = stablehlo.multiply %half, %arg0 : {T100}",
    f"    %g = stablehlo.multiply %e, %d : {T100}",
]
add("sumabs2_gelu_tanh_f32", "test/nn/activations.jl:3-33 (act = gelu, the tanh form)",
    sumabs2_module(gelu_lines, "%g"),
    [{"dims": [10, 10], "data": x_act}],
    [{"dims": [], "data": [sum((0.5 * v * (1.0 + math.tanh(c0 * (v + c1 * v ** 3)))) ** 2 for v in x_act)]}], "f32", 5e-6)

with open(os.path.join(HERE, "reactant_fixtures.json"), "w") as f:
    json.dump({"generator": "tests/golden/make_fixtures.py", "cases": cases}, f, indent=1)
print(f"wrote {len(cases)} cases")
