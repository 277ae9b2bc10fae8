"""Parser + planner on the host (no GPU): fusion decisions for the benchmark
programs and the hard-error contract for anything outside the supported set."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def kinds(plan):
    return [s["kind"] for s in plan["steps"]]


def test_sinsum_is_one_fused_map_reduce(rx):
    for raw in (False, True):
        p = rx.plan_describe(rx.programs.sinsum_add(1 << 24, raw=raw))
        assert kinds(p) == ["reduce_full"]
        s = p["steps"][0]
        assert s["chain"] == "sin_add" and s["linear"] == 1 and s["dims"] == [1 << 24]


def test_logsumexp_reads_input_once(rx):
    opt = rx.plan_describe(rx.programs.logsumexp_dims1(32768, 8192))
    assert kinds(opt) == ["logsumexp"]
    assert opt["steps"][0]["dims"][:2] == [8192, 32768]
    raw = rx.plan_describe(rx.programs.logsumexp_dims1(32768, 8192, raw=True))
    assert kinds(raw) == ["logsumexp"], "entry/exit transposes and unit-dim reshapes must fold away"


def test_jacobi_is_an_in_place_stencil_loop(rx):
    p = rx.plan_describe(rx.programs.jacobi2d(8192, 100))
    assert kinds(p) == ["loop"] and p["slots"] == 2, "no temporaries: both arrays are updated in place"
    loop = p["steps"][0]
    assert loop["trip"] == 100 and kinds(loop) if False else True
    body = loop["body"]
    assert [s["kind"] for s in body] == ["stencil"]
    assert body[0]["chain"] == "stencil5_mul" and body[0]["dims"] == [8190, 8190]


def test_jacobi_pad_select_form_plans(rx):
    p = rx.plan_describe(rx.programs.jacobi2d(64, 4, form="pad"))
    loop = [s for s in p["steps"] if s["kind"] == "loop"][0]
    assert loop["trip"] == 4
    assert any(s["kind"] == "stencil" for s in loop["body"])


def test_sharded_sinsum_gets_local_reduce_plus_all_reduce(rx):
    p = rx.plan_describe(rx.programs.sinsum_add(1 << 30, num_partitions=8))
    assert p["num_partitions"] == 8
    assert kinds(p) == ["reduce_full", "all_reduce"]
    assert p["steps"][0]["dims"] == [(1 << 30) // 8], "each device reduces its own contiguous chunk"


def test_mlp_has_five_gemms_with_folded_transposes(rx):
    p = rx.plan_describe(rx.programs.mlp_grad())
    gemms = [s["note"] for s in p["steps"] if s["kind"] == "gemm"]
    assert len(gemms) == 5
    assert sum("A(m-major)" in g for g in gemms) == 2 and sum("B(k-major)" in g for g in gemms) == 1
    assert not any(s["kind"] == "copy" for s in p["steps"])


def test_golden_modules_all_plan(rx):
    with open(os.path.join(HERE, "golden", "reactant_fixtures.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        rx.plan_describe(c["module"])   # f64 fixtures included: they plan as wide programs (tests/test_f64.py)


UNSUPPORTED = {
    "stablehlo.sort": '    %0 = "stablehlo.sort"(%arg0) ({\n    }) : (tensor<4xf32>) -> tensor<4xf32>\n    return %0 : tensor<4xf32>',
    "stablehlo.fft": "    %0 = stablehlo.fft %arg0, type = FFT, length = [4] : (tensor<4xf32>) -> tensor<4xf32>\n    return %0 : tensor<4xf32>",
    "enzymexla.kernel_call": "    %0 = enzymexla.kernel_call @k (%arg0) : (tensor<4xf32>) -> tensor<4xf32>\n    return %0 : tensor<4xf32>",
    "stablehlo.cholesky": "    %0 = stablehlo.cholesky %arg0 : tensor<4xf32>\n    return %0 : tensor<4xf32>",
}


@pytest.mark.parametrize("op", sorted(UNSUPPORTED))
def test_unsupported_op_is_a_hard_error_naming_the_op(rx, op):
    text = "module {\n  func.func @main(%arg0: tensor<4xf32>) -> tensor<4xf32> {\n" + UNSUPPORTED[op] + "\n  }\n}\n"
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(text)
    assert e.value.code == 2 and op in str(e.value)


def test_non_default_dot_precision_is_rejected(rx):
    text = rx.programs.matmul(4, 4, 4).replace("[DEFAULT, DEFAULT]", "[HIGHEST, HIGHEST]")
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(text)
    assert "HIGHEST" in str(e.value)


def test_parse_errors_carry_line_numbers(rx):
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe("module {\n  func.func @main(%arg0: tensor<4xf32>) -> tensor<4xf32> {\n    %0 = stablehlo.add %arg0, %nope : tensor<4xf32>\n    return %0 : tensor<4xf32>\n  }\n}\n")
    assert e.value.code == 1 and "line 3" in str(e.value) and "%nope" in str(e.value)


def test_dynamic_loop_bound_is_rejected(rx):
    text = """module {
  func.func @main(%arg0: tensor<4xf32>, %arg1: tensor<i64>) -> tensor<4xf32> {
    %c = stablehlo.constant dense<0> : tensor<i64>
    %c_1 = stablehlo.constant dense<1> : tensor<i64>
    %0:2 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0) : tensor<i64>, tensor<4xf32>
     cond {
      %1 = stablehlo.compare  LT, %iterArg, %arg1 : (tensor<i64>, tensor<i64>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    } do {
      %1 = stablehlo.add %iterArg, %c_1 : tensor<i64>
      %2 = stablehlo.add %iterArg_0, %iterArg_0 : tensor<4xf32>
      stablehlo.return %1, %2 : tensor<i64>, tensor<4xf32>
    }
    return %0#1 : tensor<4xf32>
  }
}
"""
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(text)
    assert "stablehlo.while" in str(e.value)


def test_maps_that_consume_a_materialised_value_join_its_producer(rx):
    """gelu activation + the bf16 operand of the next GEMM, and gelu' + its bf16 copy, are one launch each: the
    second chain reads what the first one materialised, element for element."""
    steps = rx.plan_describe(rx.programs.mlp_grad(64, 128, 32, 256))["steps"]
    notes = [s["note"] for s in steps]
    assert any("shared value %th + contraction lhs" in n for n in notes), notes
    assert any(n.startswith("shared value %dz1 + ") for n in notes), notes
    assert sum(s["kind"] == "gemm" for s in steps) == 5
    assert len(steps) == 12


def test_cumulative_reduce_window_plans_as_a_scan_and_other_windows_are_refused(rx):
    d = rx.plan_describe(rx.programs.scan((5, 4, 3), 1, "add"))
    assert [s["kind"] for s in d["steps"]] == ["scan"]
    pooling = rx.programs.scan((8, 8), 1, "maximum").replace("window_dimensions = array<i64: 1, 8>", "window_dimensions = array<i64: 1, 2>").replace(
        "[7, 0]", "[0, 0]")
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(pooling)
    assert "reduce_window" in str(e.value)
    with pytest.raises(rx.ReactantError) as e:  # the padding is filled with the init value: only the identity is accepted
        rx.plan_describe(rx.programs.scan((16,), 0, "add").replace("dense<0.000000e+00>", "dense<1.000000e+00>"))
    assert "identity" in str(e.value)


def test_reductions_over_non_adjacent_or_non_mergeable_dims_are_staged(rx):
    t = "tensor<17x3x17xf32>"
    text = f"""module {{
  func.func @main(%arg0: {t}, %arg1: tensor<3xf32>) -> (tensor<3xf32>, tensor<17x3xf32>) {{
    %z = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %b = stablehlo.broadcast_in_dim %arg1, dims = [1] : (tensor<3xf32>) -> {t}
    %0 = stablehlo.multiply %arg0, %b : {t}
    %1 = stablehlo.reduce(%0 init: %z) applies stablehlo.add across dimensions = [0, 2] : ({t}, tensor<f32>) -> tensor<3xf32>
    %2 = stablehlo.reduce(%0 init: %z) applies stablehlo.add across dimensions = [2] : ({t}, tensor<f32>) -> tensor<17x3xf32>
    return %1, %2 : tensor<3xf32>, tensor<17x3xf32>
  }}
}}
"""
    kinds = [s["kind"] for s in rx.plan_describe(text)["steps"]]
    assert kinds.count("reduce_row") + kinds.count("reduce_col") + kinds.count("reduce_full") >= 3, kinds


def test_replicated_broadcast_chain_with_several_consumers_still_meets_a_sharded_operand(rx):
    # %v2 is long and used three times; materialising it would hide that it does not vary along the sharded dim
    text = """
module attributes {mhlo.num_partitions = 2 : i64, mhlo.num_replicas = 1 : i64} {
  sdy.mesh @mesh = <["x"=2]>
  func.func @main(%arg0: tensor<516x260xf32> {sdy.sharding = #sdy.sharding<@mesh, [{"x"}, {}]>}, %arg1: tensor<260xf32> {sdy.sharding = #sdy.sharding<@mesh, [{}]>}) -> (tensor<516x260xf32> {sdy.sharding = #sdy.sharding<@mesh, [{"x"}, {}]>}) {
    %bc = stablehlo.broadcast_in_dim %arg1, dims = [1] : (tensor<260xf32>) -> tensor<516x260xf32>
    %t0 = stablehlo.tanh %bc : tensor<516x260xf32>
    %v0 = stablehlo.multiply %bc, %t0 : tensor<516x260xf32>
    %v1 = stablehlo.maximum %v0, %bc : tensor<516x260xf32>
    %t2 = stablehlo.tanh %bc : tensor<516x260xf32>
    %v2 = stablehlo.multiply %v1, %t2 : tensor<516x260xf32>
    %t3 = stablehlo.tanh %v2 : tensor<516x260xf32>
    %v3 = stablehlo.multiply %v2, %t3 : tensor<516x260xf32>
    %t5 = stablehlo.tanh %arg0 : tensor<516x260xf32>
    %v5 = stablehlo.multiply %v3, %t5 : tensor<516x260xf32>
    %v6 = stablehlo.subtract %v5, %v2 : tensor<516x260xf32>
    return %v6 : tensor<516x260xf32>
  }
}
"""
    d = rx.plan_describe(text)
    assert [s["kind"] for s in d["steps"]] == ["map"], d["steps"]
    assert d["steps"][0]["dims"] == [258, 260] or d["steps"][0]["dims"] == [258 * 260], d["steps"]


def test_reduce_over_a_sharded_dim_of_local_extent_one_still_crosses_the_mesh(rx):
    text = """
module attributes {mhlo.num_partitions = 2 : i64, mhlo.num_replicas = 1 : i64} {
  sdy.mesh @mesh = <["x"=2]>
  func.func @main(%arg0: tensor<260x2xf32> {sdy.sharding = #sdy.sharding<@mesh, [{}, {"x"}]>}) -> tensor<260xf32> {
    %s = stablehlo.sine %arg0 : tensor<260x2xf32>
    %z = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %red = stablehlo.reduce(%s init: %z) applies stablehlo.add across dimensions = [1] : (tensor<260x2xf32>, tensor<f32>) -> tensor<260xf32>
    return %red : tensor<260xf32>
  }
}
"""
    kinds = [s["kind"] for s in rx.plan_describe(text)["steps"]]
    assert kinds == ["map", "all_reduce"], kinds


def test_sharded_reduce_applies_a_nonzero_init_once(rx):
    """sum over the mesh of (local sum + init) would count init once per device: the local reduce must start from
    the identity and the init value be added after the all-reduce."""
    text = rx.programs.sinsum_add(1 << 12, num_partitions=4).replace("dense<0.000000e+00> : tensor<f32>", "dense<5.000000e+00> : tensor<f32>")
    p = rx.plan_describe(text)
    assert kinds(p) == ["reduce_full", "all_reduce", "map"], p
    assert "after the all-reduce" in p["steps"][2]["note"]
    # unsharded: the init value is folded into the reduce itself, no extra step
    p1 = rx.plan_describe(rx.programs.sinsum_add(1 << 12).replace("dense<0.000000e+00> : tensor<f32>", "dense<5.000000e+00> : tensor<f32>"))
    assert kinds(p1) == ["reduce_full"]


def test_jacobi_two_half_steps_plan_in_place_without_a_copy(rx):
    """benchmark/polybench/stencil.jl:263-289 updates B from A and then A from B inside one iteration.  When the
    second update is planned, the slices of A have already been consumed by the first (emitted) step, so A may be
    written in place: two stencil steps, two slots, no copy."""
    p = rx.plan_describe(rx.programs.jacobi2d(8192, 50, form="halfsteps"))
    assert kinds(p) == ["loop"] and p["slots"] == 2
    body = p["steps"][0]["body"]
    assert [s["kind"] for s in body] == ["stencil", "stencil"] and all(s["chain"] == "stencil5_mul" for s in body)


def test_nested_concatenates_around_an_update_plan_as_the_update_in_place(rx):
    """The concatenate spelling of a window update (borders of B's rows around the new interior, then B's first and
    last row around that) plans exactly like the dynamic_update_slice it was rewritten from: the inner concatenate is
    not materialised, the border pieces already sit where they belong, and the interior is written into B."""
    p = rx.plan_describe(rx.programs.jacobi2d(8192, 100, form="concat"))
    q = rx.plan_describe(rx.programs.jacobi2d(8192, 100, form="dus"))
    assert kinds(p) == ["loop"] and p["slots"] == q["slots"] == 2
    body = p["steps"][0]["body"]
    assert [s["kind"] for s in body] == ["stencil"] and body[0]["chain"] == "stencil5_mul", body
    # when the old array is still read afterwards the pieces are written into a fresh array instead
    t = "tensor<8x8xf32>"
    text = f"""module {{
  func.func @main(%arg0: {t} {{tf.aliasing_output = 0 : i32}}, %arg1: tensor<6x8xf32>) -> ({t}, {t}) {{
    %top = stablehlo.slice %arg0 [0:1, 0:8] : ({t}) -> tensor<1x8xf32>
    %bot = stablehlo.slice %arg0 [7:8, 0:8] : ({t}) -> tensor<1x8xf32>
    %0 = stablehlo.concatenate %top, %arg1, %bot, dim = 0 : (tensor<1x8xf32>, tensor<6x8xf32>, tensor<1x8xf32>) -> {t}
    %1 = stablehlo.sine %arg0 : {t}
    return %0, %1 : {t}, {t}
  }}
}}
"""
    k = kinds(rx.plan_describe(text))
    assert k.count("map") == 4, k   # three pieces into a new array + the sine
    # a piece taken from somewhere else in the target is not "in place"
    text2 = text.replace("[7:8, 0:8]", "[6:7, 0:8]").replace("    %1 = stablehlo.sine %arg0 : " + t + "\n", "").replace("return %0, %1 : " + t + ", " + t, "return %0 : " + t).replace(f"-> ({t}, {t})", f"-> {t}")
    assert kinds(rx.plan_describe(text2)).count("map") == 3


def test_pad_and_select_around_an_update_plan_as_the_update_in_place(rx, ref):
    """The pad + select spelling of a window update -- select(mask, pad(update), target) with mask = `true` padded
    with `false` by the same amounts -- plans like the dynamic_update_slice it was rewritten from: the padded update
    is not materialised and the loop body is the one stencil step.  A mask that does not match the padding, or a
    padded update that something else reads too, keeps the general plan (pad into a new array, select as a map)."""
    p = rx.plan_describe(rx.programs.jacobi2d(8192, 100, form="pad"))
    loop = [s for s in p["steps"] if s["kind"] == "loop"]
    assert len(loop) == 1 and [s["kind"] for s in loop[0]["body"]] == ["stencil"], p["steps"]
    assert loop[0]["body"][0]["chain"] == "stencil5_mul"
    t, ti, tm = "tensor<8x8xf32>", "tensor<6x6xf32>", "tensor<8x8xi1>"
    text = f"""module {{
  func.func @main(%arg0: {t} {{tf.aliasing_output = 0 : i32}}, %arg1: {ti}) -> {t} {{
    %z = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %false = stablehlo.constant dense<false> : tensor<i1>
    %ones = stablehlo.constant dense<true> : tensor<6x6xi1>
    %pm = stablehlo.pad %ones, %false, low = [1, 1], high = [1, 1], interior = [0, 0] : (tensor<6x6xi1>, tensor<i1>) -> {tm}
    %pu = stablehlo.pad %arg1, %z, low = [1, 1], high = [1, 1], interior = [0, 0] : ({ti}, tensor<f32>) -> {t}
    %0 = stablehlo.select %pm, %pu, %arg0 : {tm}, {t}
    return %0 : {t}
  }}
}}
"""
    notes = [s.get("note", "") for s in rx.plan_describe(text)["steps"]]
    assert any("update window at offset 9" in n for n in notes) and not any("pad interior" in n and "f32" in n for n in notes[2:]), notes
    x = np.arange(64, dtype=np.float32).reshape(8, 8)
    u = -np.arange(36, dtype=np.float32).reshape(6, 6)
    want = x.copy()
    want[1:7, 1:7] = u
    assert np.array_equal(ref.run_module(text, [x, u])[0], want)
    # the update padded differently from the mask: not a window update
    other = text.replace("%pu = stablehlo.pad %arg1, %z, low = [1, 1], high = [1, 1]", "%pu = stablehlo.pad %arg1, %z, low = [2, 1], high = [0, 1]")
    notes = [s.get("note", "") for s in rx.plan_describe(other)["steps"]]
    assert not any("update window" in n for n in notes), notes


def test_update_target_that_is_still_read_later_is_copied(rx):
    """In place only when nothing still to be evaluated reads the target: here the old array is returned too."""
    t, ti = "tensor<8x8xf32>", "tensor<6x6xf32>"
    text = f"""module {{
  func.func @main(%arg0: {t} {{tf.aliasing_output = 0 : i32}}, %arg1: {ti}) -> ({t}, {t}) {{
    %c = stablehlo.constant dense<1> : tensor<i32>
    %0 = stablehlo.dynamic_update_slice %arg0, %arg1, %c, %c : ({t}, {ti}, tensor<i32>, tensor<i32>) -> {t}
    %1 = stablehlo.sine %arg0 : {t}
    return %0, %1 : {t}, {t}
  }}
}}
"""
    p = rx.plan_describe(text)
    assert "copy" in kinds(p), p


def test_row_sharded_jacobi_plans_with_halo_rows(rx):
    for form, body in (("dus", ["stencil"]), ("halfsteps", ["stencil", "stencil"])):
        p = rx.plan_describe(rx.programs.jacobi2d(8192, 100, form=form, num_partitions=8))
        assert kinds(p) == ["rows_in", "rows_in", "loop", "rows_out", "rows_out"]
        loop = p["steps"][2]
        assert [s["kind"] for s in loop["body"]] == body and "halo 2 up, 2 down" in loop["note"]
    # a loop that carries anything else in sharded form is refused by name
    text = rx.programs.jacobi1d(64, 2).replace("mhlo.num_partitions = 1", "mhlo.num_partitions = 2")
    text = text.replace("  func.func @main", '  sdy.mesh @mesh = <["x"=2]>\n  func.func @main', 1)
    text = text.replace("{tf.aliasing_output = 0 : i32}", '{tf.aliasing_output = 0 : i32, sdy.sharding = #sdy.sharding<@mesh, [{"x"}]>}')
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(text)
    assert e.value.code == 2 and "sharded" in str(e.value)


def test_a_dimension_the_mesh_does_not_divide_is_replicated(rx):
    """src/Sharding.jl:582-654: no padding; the argument falls back to a sharding that fits -- here replication, so the
    reduce needs no all-reduce and every device computes the whole sum."""
    p = rx.plan_describe(rx.programs.sinsum_add(1001, num_partitions=4))
    assert kinds(p) == ["reduce_full"] and p["steps"][0]["dims"] == [1001]
