"""StableHLO module text for the benchmark configurations, in the form Reactant
hands to its runtime: `func.func @main` over reversed-dim tensors, printed by
MLIR's default printer.

Reactant's tracer and pass pipeline cannot run where this engine is built (no
Julia), so these are written out by hand from the op emitters:
  sum / maximum  -> stablehlo.reduce       src/TracedRArray.jl:187-230, src/Ops.jl:3491-3622
  broadcasting   -> elementwise ops        src/TracedUtils.jl:1202-1352
  A[r, c]        -> stablehlo.slice        src/Indexing.jl:552-627, src/Ops.jl:761-793
  B[r, c] = v    -> dynamic_update_slice   src/Indexing.jl:350-446, src/Ops.jl:3662-3678
  @trace for     -> stablehlo.while        src/Ops.jl:2349-2447
  W * X          -> stablehlo.dot_general  src/stdlibs/LinearAlgebra.jl:274-330
  sharding attrs -> sdy.mesh / sdy.sharding src/Sharding.jl:512-575
Each generator offers the optimised form (`raw=False`: layout transposes already
propagated away) and, where it differs, the raw trace form (`raw=True`: every
argument and result wrapped in the reversed-dims transposes of
src/TracedUtils.jl:608-626).
"""
from __future__ import annotations

import math


def _t(shape, et="f32"):
    return "tensor<" + "".join(f"{d}x" for d in shape) + et + ">"


def sinsum_add(n: int, raw: bool = False, num_partitions: int = 1) -> str:
    """f(x, y) = sum(sin.(x) .+ y) on Float32 vectors of length n.
    With num_partitions > 1 both vectors are sharded along a 1-D mesh "x"."""
    t = _t([n])
    shard = ' {sdy.sharding = #sdy.sharding<@mesh, [{"x"}]>}' if num_partitions > 1 else ""
    mesh = f'  sdy.mesh @mesh = <["x"={num_partitions}]>\n' if num_partitions > 1 else ""
    body = []
    x, y = "%arg0", "%arg1"
    if raw:
        body.append(f"    %t0 = stablehlo.transpose %arg0, dims = [0] : ({t}) -> {t}")
        body.append(f"    %t1 = stablehlo.transpose %arg1, dims = [0] : ({t}) -> {t}")
        x, y = "%t0", "%t1"
    body += [
        "    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>",
        f"    %0 = stablehlo.sine {x} : {t}",
        f"    %1 = stablehlo.add %0, {y} : {t}",
        f"    %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [0] : ({t}, tensor<f32>) -> tensor<f32>",
        "    return %2 : tensor<f32>",
    ]
    return (f"module @reactant_sinsum_add attributes {{mhlo.num_partitions = {num_partitions} : i64, mhlo.num_replicas = 1 : i64}} {{\n"
            f"{mesh}  func.func @main(%arg0: {t}{shard}, %arg1: {t}{shard}) -> tensor<f32> {{\n" + "\n".join(body) + "\n  }\n}\n")


def logsumexp_dims1(rows: int, cols: int, raw: bool = False) -> str:
    """m = maximum(x; dims=1); m .+ log.(sum(exp.(x .- m); dims=1)) for a Julia
    rows x cols Float32 matrix (argument tensor is cols x rows)."""
    ta, tc, tr = _t([cols, rows]), _t([cols]), _t([cols, 1])
    if not raw:
        body = f"""    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %cst_0 = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %0 = stablehlo.reduce(%arg0 init: %cst_0) applies stablehlo.maximum across dimensions = [1] : ({ta}, tensor<f32>) -> {tc}
    %1 = stablehlo.broadcast_in_dim %0, dims = [0] : ({tc}) -> {ta}
    %2 = stablehlo.subtract %arg0, %1 : {ta}
    %3 = stablehlo.exponential %2 : {ta}
    %4 = stablehlo.reduce(%3 init: %cst) applies stablehlo.add across dimensions = [1] : ({ta}, tensor<f32>) -> {tc}
    %5 = stablehlo.log %4 : {tc}
    %6 = stablehlo.add %0, %5 : {tc}
    %7 = stablehlo.reshape %6 : ({tc}) -> {tr}
    return %7 : {tr}"""
    else:
        tl, t1 = _t([rows, cols]), _t([1, cols])
        body = f"""    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %cst_0 = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %0 = stablehlo.transpose %arg0, dims = [1, 0] : ({ta}) -> {tl}
    %1 = stablehlo.reduce(%0 init: %cst_0) applies stablehlo.maximum across dimensions = [0] : ({tl}, tensor<f32>) -> {tc}
    %2 = stablehlo.reshape %1 : ({tc}) -> {t1}
    %3 = stablehlo.broadcast_in_dim %2, dims = [0, 1] : ({t1}) -> {tl}
    %4 = stablehlo.subtract %0, %3 : {tl}
    %5 = stablehlo.exponential %4 : {tl}
    %6 = stablehlo.reduce(%5 init: %cst) applies stablehlo.add across dimensions = [0] : ({tl}, tensor<f32>) -> {tc}
    %7 = stablehlo.reshape %6 : ({tc}) -> {t1}
    %8 = stablehlo.log %7 : {t1}
    %9 = stablehlo.add %2, %8 : {t1}
    %10 = stablehlo.transpose %9, dims = [1, 0] : ({t1}) -> {tr}
    return %10 : {tr}"""
    return ("module @reactant_logsumexp attributes {mhlo.num_partitions = 1 : i64, mhlo.num_replicas = 1 : i64} {\n"
            f"  func.func @main(%arg0: {ta}) -> {tr} {{\n{body}\n  }}\n}}\n")


def jacobi2d(n: int, steps: int, form: str = "dus", num_partitions: int = 1) -> str:
    """Jacobi-2D on n x n Float32 arrays; both arrays are mutated, hence donated and aliased to the two results.

    form="dus" / "pad": `steps` sweeps of
        B[2:end-1,2:end-1] = 0.2f0 .* (A[c] .+ A[i-1] .+ A[i+1] .+ A[j-1] .+ A[j+1]); A, B = B, A
    with the interior written by dynamic_update_slice ("dus") or by the pad + select rewrite that Enzyme-JAX's
    communication patterns can produce ("pad", src/compiler/OptimizationPasses.jl:356-372).
    form="concat": the same update with the interior placed by two nested concatenates -- the borders of B's rows
    around the new interior, then B's first and last row around that -- which is what the rewrite of a
    dynamic_update_slice into concatenates leaves (src/CompileOptions.jl:22-41).
    form="halfsteps": the spelling of benchmark/polybench/stencil.jl:263-289 -- every one of the `steps`
    iterations updates B from A and then A from B (two sweeps, no swap), the five terms added in that file's
    order: centre, j-1, j+1, i+1, i-1.
    With num_partitions > 1 both arrays are split over a 1-D mesh along Julia's second dimension (the first, i.e.
    row, dimension of the tensors): NamedSharding(mesh, (nothing, :x))."""
    t, ti = _t([n, n]), _t([n - 2, n - 2])
    shard = ', sdy.sharding = #sdy.sharding<@mesh, [{"x"}, {}]>' if num_partitions > 1 else ""
    mesh = f'  sdy.mesh @mesh = <["x"={num_partitions}]>\n' if num_partitions > 1 else ""
    m = n - 1
    # physical dims are reversed Julia dims: Julia A[i-1, j] is the minor-dim neighbour
    centre, i_lo, i_hi, j_lo, j_hi = f"[1:{m}, 1:{m}]", f"[1:{m}, 0:{n - 2}]", f"[1:{m}, 2:{n}]", f"[0:{n - 2}, 1:{m}]", f"[2:{n}, 1:{m}]"

    def sweep(src, tag, order):
        out = [f"      %s{tag}{k} = stablehlo.slice {src} {sl} : ({t}) -> {ti}" for k, sl in enumerate(order)]
        out += [
            f"      %a{tag}0 = stablehlo.add %s{tag}0, %s{tag}1 : {ti}",
            f"      %a{tag}1 = stablehlo.add %a{tag}0, %s{tag}2 : {ti}",
            f"      %a{tag}2 = stablehlo.add %a{tag}1, %s{tag}3 : {ti}",
            f"      %a{tag}3 = stablehlo.add %a{tag}2, %s{tag}4 : {ti}",
            f"      %u{tag} = stablehlo.multiply %cst, %a{tag}3 : {ti}",
        ]
        return out

    dus = lambda dst, upd, res: f"      {res} = stablehlo.dynamic_update_slice {dst}, {upd}, %c_1, %c_1 : ({t}, {ti}, tensor<i32>, tensor<i32>) -> {t}"
    extra = ""
    if form == "halfsteps":
        order = [centre, j_lo, j_hi, i_hi, i_lo]
        lines = sweep("%iterArg_0", "p", order) + [dus("%iterArg_1", "%up", "%nb")] + sweep("%nb", "q", order) + [dus("%iterArg_0", "%uq", "%na")]
        yields = "%1, %na, %nb"
    else:
        lines = sweep("%iterArg_0", "", [centre, i_lo, i_hi, j_lo, j_hi])
        if form == "dus":
            lines.append(dus("%iterArg_1", "%u", "%nb"))
        elif form == "concat":
            tc, tr, tm = _t([n - 2, 1]), _t([1, n]), _t([n - 2, n])
            lines += [
                f"      %left = stablehlo.slice %iterArg_1 [1:{m}, 0:1] : ({t}) -> {tc}",
                f"      %right = stablehlo.slice %iterArg_1 [1:{m}, {m}:{n}] : ({t}) -> {tc}",
                f"      %mid = stablehlo.concatenate %left, %u, %right, dim = 1 : ({tc}, {ti}, {tc}) -> {tm}",
                f"      %top = stablehlo.slice %iterArg_1 [0:1, 0:{n}] : ({t}) -> {tr}",
                f"      %bot = stablehlo.slice %iterArg_1 [{m}:{n}, 0:{n}] : ({t}) -> {tr}",
                f"      %nb = stablehlo.concatenate %top, %mid, %bot, dim = 0 : ({tr}, {tm}, {tr}) -> {t}",
            ]
        else:
            lines += [
                f"      %pu = stablehlo.pad %u, %cst_z, low = [1, 1], high = [1, 1], interior = [0, 0] : ({ti}, tensor<f32>) -> {t}",
                f"      %nb = stablehlo.select %pm, %pu, %iterArg_1 : {_t([n, n], 'i1')}, {t}",
            ]
            extra = (f"    %cst_z = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
                     f"    %false = stablehlo.constant dense<false> : tensor<i1>\n"
                     f"    %ones = stablehlo.constant dense<true> : {_t([n - 2, n - 2], 'i1')}\n"
                     f"    %pm = stablehlo.pad %ones, %false, low = [1, 1], high = [1, 1], interior = [0, 0] : ({_t([n - 2, n - 2], 'i1')}, tensor<i1>) -> {_t([n, n], 'i1')}\n")
        yields = "%1, %nb, %iterArg_0"
    body = "\n".join(lines)
    return f"""module @reactant_jacobi2d attributes {{mhlo.num_partitions = {num_partitions} : i64, mhlo.num_replicas = 1 : i64}} {{
{mesh}  func.func @main(%arg0: {t} {{tf.aliasing_output = 0 : i32{shard}}}, %arg1: {t} {{tf.aliasing_output = 1 : i32{shard}}}) -> ({t}, {t}) {{
    %c = stablehlo.constant dense<0> : tensor<i64>
    %c_0 = stablehlo.constant dense<{steps}> : tensor<i64>
    %c_2 = stablehlo.constant dense<1> : tensor<i64>
    %c_1 = stablehlo.constant dense<1> : tensor<i32>
    %cst = stablehlo.constant dense<2.000000e-01> : {ti}
{extra}    %0:3 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0, %iterArg_1 = %arg1) : tensor<i64>, {t}, {t} attributes {{enzyme.disable_mincut}}
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


def mlp_grad(features: int = 1024, hidden: int = 4096, out: int = 1024, batch: int = 4096, num_partitions: int = 1) -> str:
    """Two-layer MLP forward + reverse-mode gradient, as it reaches the runtime
    after Enzyme's pass has synthesised the reverse program: five dot_generals
    (two forward, three transposed-operand backward), gelu(tanh) and its
    derivative as elementwise chains, bias gradients as column reductions.

    Julia shapes: W1 hidden x features (bf16), b1 hidden (f32), W2 out x hidden
    (bf16), b2 out (f32), X features x batch (bf16), Y out x batch (f32).
    Results: dW1, db1, dW2, db2, loss.

    With num_partitions > 1 the batch is split over a 1-D mesh (data parallelism): X and Y carry
    `sdy.sharding` on their batch dimension, the weights are replicated, and every gradient is a
    sum over devices, so the runtime has to all-reduce them.
    """
    F, H, O, B = features, hidden, out, batch
    tW1, tW2, tX, tY = _t([F, H], "bf16"), _t([H, O], "bf16"), _t([B, F], "bf16"), _t([B, O])
    tb1, tb2 = _t([H]), _t([O])
    tZ1b, tZ1 = _t([B, H], "bf16"), _t([B, H])
    tZ2b, tZ2 = _t([B, O], "bf16"), _t([B, O])
    c = math.sqrt(2.0 / math.pi)
    inv = 1.0 / (B * O)

    def k(v, t):
        return f"stablehlo.constant dense<{v:.9e}> : {t}"

    sh = ' {sdy.sharding = #sdy.sharding<@mesh, [{"x"}, {}]>}' if num_partitions > 1 else ""
    mesh = f'  sdy.mesh @mesh = <["x"={num_partitions}]>\n' if num_partitions > 1 else ""
    return f"""module @reactant_mlp_grad attributes {{mhlo.num_partitions = {num_partitions} : i64, mhlo.num_replicas = 1 : i64}} {{
{mesh}  func.func @main(%arg0: {tW1}, %arg1: {tb1}, %arg2: {tW2}, %arg3: {tb2}, %arg4: {tX}{sh}, %arg5: {tY}{sh}) -> ({tW1}, {tb1}, {tW2}, {tb2}, tensor<f32>) {{
    %zero = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %half = {k(0.5, tZ1)}
    %one = {k(1.0, tZ1)}
    %ca = {k(0.044715, tZ1)}
    %c3a = {k(3 * 0.044715, tZ1)}
    %cc = {k(c, tZ1)}
    %cinv = {k(inv, "tensor<f32>")}
    %c2inv = {k(2 * inv, tZ2)}
    %0 = stablehlo.dot_general %arg4, %arg0, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : ({tX}, {tW1}) -> {tZ1b}
    %1 = stablehlo.convert %0 : ({tZ1b}) -> {tZ1}
    %2 = stablehlo.broadcast_in_dim %arg1, dims = [1] : ({tb1}) -> {tZ1}
    %z1 = stablehlo.add %1, %2 : {tZ1}
    %z1sq = stablehlo.multiply %z1, %z1 : {tZ1}
    %z1cu = stablehlo.multiply %z1sq, %z1 : {tZ1}
    %3 = stablehlo.multiply %ca, %z1cu : {tZ1}
    %4 = stablehlo.add %z1, %3 : {tZ1}
    %5 = stablehlo.multiply %cc, %4 : {tZ1}
    %th = stablehlo.tanh %5 : {tZ1}
    %6 = stablehlo.add %one, %th : {tZ1}
    %7 = stablehlo.multiply %half, %z1 : {tZ1}
    %h = stablehlo.multiply %7, %6 : {tZ1}
    %hb = stablehlo.convert %h : ({tZ1}) -> {tZ1b}
    %8 = stablehlo.dot_general %hb, %arg2, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : ({tZ1b}, {tW2}) -> {tZ2b}
    %9 = stablehlo.convert %8 : ({tZ2b}) -> {tZ2}
    %10 = stablehlo.broadcast_in_dim %arg3, dims = [1] : ({tb2}) -> {tZ2}
    %z2 = stablehlo.add %9, %10 : {tZ2}
    %d = stablehlo.subtract %z2, %arg5 : {tZ2}
    %dd = stablehlo.multiply %d, %d : {tZ2}
    %11 = stablehlo.reduce(%dd init: %zero) applies stablehlo.add across dimensions = [0, 1] : ({tZ2}, tensor<f32>) -> tensor<f32>
    %loss = stablehlo.multiply %11, %cinv : tensor<f32>
    %dz2 = stablehlo.multiply %c2inv, %d : {tZ2}
    %db2 = stablehlo.reduce(%dz2 init: %zero) applies stablehlo.add across dimensions = [0] : ({tZ2}, tensor<f32>) -> {tb2}
    %dz2b = stablehlo.convert %dz2 : ({tZ2}) -> {tZ2b}
    %dw2 = stablehlo.dot_general %hb, %dz2b, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : ({tZ1b}, {tZ2b}) -> {tW2}
    %dhb = stablehlo.dot_general %dz2b, %arg2, contracting_dims = [1] x [1], precision = [DEFAULT, DEFAULT] : ({tZ2b}, {tW2}) -> {tZ1b}
    %dh = stablehlo.convert %dhb : ({tZ1b}) -> {tZ1}
    %12 = stablehlo.multiply %th, %th : {tZ1}
    %13 = stablehlo.subtract %one, %12 : {tZ1}
    %14 = stablehlo.multiply %c3a, %z1sq : {tZ1}
    %15 = stablehlo.add %one, %14 : {tZ1}
    %16 = stablehlo.multiply %cc, %15 : {tZ1}
    %17 = stablehlo.multiply %13, %16 : {tZ1}
    %18 = stablehlo.multiply %7, %17 : {tZ1}
    %19 = stablehlo.multiply %half, %6 : {tZ1}
    %gp = stablehlo.add %19, %18 : {tZ1}
    %dz1 = stablehlo.multiply %dh, %gp : {tZ1}
    %db1 = stablehlo.reduce(%dz1 init: %zero) applies stablehlo.add across dimensions = [0] : ({tZ1}, tensor<f32>) -> {tb1}
    %dz1b = stablehlo.convert %dz1 : ({tZ1}) -> {tZ1b}
    %dw1 = stablehlo.dot_general %arg4, %dz1b, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : ({tX}, {tZ1b}) -> {tW1}
    return %dw1, %db1, %dw2, %db2, %loss : {tW1}, {tb1}, {tW2}, {tb2}, tensor<f32>
  }}
}}
"""


def matmul(m: int, k: int, n: int, et: str = "f32") -> str:
    """C = A * B for Julia A (m x k), B (k x n): the arguments arrive as k x m and
    n x k tensors and the product as n x m (test/core/compile.jl:350-355)."""
    ta, tb, tc = _t([k, m], et), _t([n, k], et), _t([n, m], et)
    return f"""module @reactant_matmul attributes {{mhlo.num_partitions = 1 : i64, mhlo.num_replicas = 1 : i64}} {{
  func.func @main(%arg0: {ta}, %arg1: {tb}) -> {tc} {{
    %0 = stablehlo.dot_general %arg1, %arg0, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : ({tb}, {ta}) -> {tc}
    return %0 : {tc}
  }}
}}
"""


def scan(xla_dims, xla_axis: int, kind: str = "add", et: str = "f32") -> str:
    """cumsum / cumprod / accumulate(max|min) along one dimension, as Reactant's scan_impl! lowers it
    (src/TracedRArray.jl:1049-1107): stablehlo.reduce_window whose window is the whole dimension, padded low by
    its extent minus one, with the combiner's identity as init value.  `xla_dims` are the boundary (reversed)
    dims; Julia `dims = d` of an N-d array is boundary dim N - d."""
    rank = len(xla_dims)
    win = [1] * rank
    win[xla_axis] = xla_dims[xla_axis]
    pads = "[" + ", ".join(f"[{xla_dims[d] - 1 if d == xla_axis else 0}, 0]" for d in range(rank)) + "]"
    ones = ", ".join(["1"] * rank)
    flt = et in ("f32", "bf16")
    init = {"add": "0.000000e+00" if flt else "0", "multiply": "1.000000e+00" if flt else "1",
            "maximum": "0xFF800000" if flt else "-2147483648", "minimum": "0x7F800000" if flt else "2147483647"}[kind]
    ty, sc = _t(list(xla_dims), et), _t([], et)
    return f"""module @reactant_scan attributes {{mhlo.num_partitions = 1 : i64, mhlo.num_replicas = 1 : i64}} {{
  func.func @main(%arg0: {ty}) -> {ty} {{
    %cst = stablehlo.constant dense<{init}> : {sc}
    %0 = "stablehlo.reduce_window"(%arg0, %cst) <{{base_dilations = array<i64: {ones}>, padding = dense<{pads}> : tensor<{rank}x2xi64>, window_dilations = array<i64: {ones}>, window_dimensions = array<i64: {', '.join(map(str, win))}>, window_strides = array<i64: {ones}>}}> ({{
    ^bb0(%arg1: {sc}, %arg2: {sc}):
      %1 = stablehlo.{kind} %arg1, %arg2 : {sc}
      stablehlo.return %1 : {sc}
    }}) : ({ty}, {sc}) -> {ty}
    return %0 : {ty}
  }}
}}
"""


class _Body:
    """Emits the ops of a loop body line by line, naming results %v0, %v1, ..."""

    def __init__(self):
        self.lines, self.n = [], 0

    def op(self, text, ty):
        name = f"%v{self.n}"
        self.n += 1
        self.lines.append(f"      {name} = {text} : {ty}")
        return name

    def slice(self, src, ranges, t_in, t_out):
        name = f"%v{self.n}"
        self.n += 1
        spec = ", ".join(f"{a}:{b}" for a, b in ranges)
        self.lines.append(f"      {name} = stablehlo.slice {src} [{spec}] : ({t_in}) -> {t_out}")
        return name

    def dus(self, dst, upd, starts, t, tu):
        name = f"%v{self.n}"
        self.n += 1
        idx = ", ".join(starts)
        types = ", ".join([t, tu] + ["tensor<i32>"] * len(starts))
        self.lines.append(f"      {name} = stablehlo.dynamic_update_slice {dst}, {upd}, {idx} : ({types}) -> {t}")
        return name


def _two_array_loop(name, shape, steps, consts, body_lines, yield_a, yield_b):
    t = _t(shape)
    cs = "\n".join(f"    {n} = stablehlo.constant dense<{v}> : {ty}" for n, v, ty in consts)
    body = "\n".join(body_lines)
    return f"""module @reactant_{name} attributes {{mhlo.num_partitions = 1 : i64, mhlo.num_replicas = 1 : i64}} {{
  func.func @main(%arg0: {t} {{tf.aliasing_output = 0 : i32}}, %arg1: {t} {{tf.aliasing_output = 1 : i32}}) -> ({t}, {t}) {{
    %c = stablehlo.constant dense<0> : tensor<i64>
    %c_0 = stablehlo.constant dense<{steps}> : tensor<i64>
    %c_2 = stablehlo.constant dense<1> : tensor<i64>
    %c_1 = stablehlo.constant dense<1> : tensor<i32>
{cs}
    %0:3 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0, %iterArg_1 = %arg1) : tensor<i64>, {t}, {t} attributes {{enzyme.disable_mincut}}
     cond {{
      %1 = stablehlo.compare  LT, %iterArg, %c_0 : (tensor<i64>, tensor<i64>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    }} do {{
      %1 = stablehlo.add %iterArg, %c_2 : tensor<i64>
{body}
      stablehlo.return %1, {yield_a}, {yield_b} : tensor<i64>, {t}, {t}
    }}
    return %0#1, %0#2 : {t}, {t}
  }}
}}
"""


def fdtd2d(nx: int, ny: int, tmax: int) -> str:
    """benchmark/polybench/stencil.jl:42-72 (fdtd_2d_vectorized): per time step t
        EY[1, :] .= fict[t]
        EY[2:NX, :]       .-= 0.5 .* (HZ[2:NX, :] .- HZ[1:NX-1, :])
        EX[:, 2:NY]       .-= 0.5 .* (HZ[:, 2:NY] .- HZ[:, 1:NY-1])
        HZ[1:NX-1,1:NY-1] .-= 0.7 .* (EX[1:NX-1,2:NY] .- EX[1:NX-1,1:NY-1] .+ EY[2:NX,1:NY-1] .- EY[1:NX-1,1:NY-1])
    on NX x NY Float32 arrays (tensors [NY][NX]).  `fict[t]` is a scalar read at the traced loop variable: the
    induction value start + i * step of the counter (src/ControlFlow / ReactantCore `@trace for`), converted to Int32 and
    made 0-based (src/Ops.jl:3624-3646), a dynamic_slice of one element (src/Indexing.jl:25-31) reshaped to a scalar and
    broadcast into the first row.  All three arrays are mutated, hence donated and returned."""
    t, tf = _t([ny, nx]), _t([tmax])
    b = _Body()
    ti = b.op("stablehlo.multiply %iterArg, %c_2", "tensor<i64>")
    ti = b.op(f"stablehlo.add {ti}, %c_2", "tensor<i64>")
    t32 = f"%v{b.n}"
    b.n += 1
    b.lines.append(f"      {t32} = stablehlo.convert {ti} : (tensor<i64>) -> tensor<i32>")
    idx = b.op(f"stablehlo.subtract {t32}, %c_1", "tensor<i32>")
    fs = f"%v{b.n}"
    b.n += 1
    b.lines.append(f"      {fs} = stablehlo.dynamic_slice %arg3, {idx}, sizes = [1] : ({tf}, tensor<i32>) -> tensor<1xf32>")
    f0 = f"%v{b.n}"
    b.n += 1
    b.lines.append(f"      {f0} = stablehlo.reshape {fs} : (tensor<1xf32>) -> tensor<f32>")
    tcol = _t([ny, 1])
    row = f"%v{b.n}"
    b.n += 1
    b.lines.append(f"      {row} = stablehlo.broadcast_in_dim {f0}, dims = [] : (tensor<f32>) -> {tcol}")
    ey1 = b.dus("%iterArg_1", row, ["%c_z", "%c_z"], t, tcol)
    # EY[2:NX, :]: tensor columns 1..NX-1
    te = _t([ny, nx - 1])
    a = b.slice(ey1, [(0, ny), (1, nx)], t, te)
    h1 = b.slice("%iterArg_2", [(0, ny), (1, nx)], t, te)
    h0 = b.slice("%iterArg_2", [(0, ny), (0, nx - 1)], t, te)
    d = b.op(f"stablehlo.subtract {h1}, {h0}", te)
    mm = b.op(f"stablehlo.multiply %half_e, {d}", te)
    u = b.op(f"stablehlo.subtract {a}, {mm}", te)
    ey2 = b.dus(ey1, u, ["%c_z", "%c_1"], t, te)
    # EX[:, 2:NY]: tensor rows 1..NY-1
    tx = _t([ny - 1, nx])
    a = b.slice("%iterArg_0", [(1, ny), (0, nx)], t, tx)
    h1 = b.slice("%iterArg_2", [(1, ny), (0, nx)], t, tx)
    h0 = b.slice("%iterArg_2", [(0, ny - 1), (0, nx)], t, tx)
    d = b.op(f"stablehlo.subtract {h1}, {h0}", tx)
    mm = b.op(f"stablehlo.multiply %half_x, {d}", tx)
    u = b.op(f"stablehlo.subtract {a}, {mm}", tx)
    ex2 = b.dus("%iterArg_0", u, ["%c_1", "%c_z"], t, tx)
    # HZ[1:NX-1, 1:NY-1]
    th = _t([ny - 1, nx - 1])
    hz = b.slice("%iterArg_2", [(0, ny - 1), (0, nx - 1)], t, th)
    x1 = b.slice(ex2, [(1, ny), (0, nx - 1)], t, th)
    x0 = b.slice(ex2, [(0, ny - 1), (0, nx - 1)], t, th)
    y1 = b.slice(ey2, [(0, ny - 1), (1, nx)], t, th)
    y0 = b.slice(ey2, [(0, ny - 1), (0, nx - 1)], t, th)
    s1 = b.op(f"stablehlo.subtract {x1}, {x0}", th)
    s2 = b.op(f"stablehlo.add {s1}, {y1}", th)
    s3 = b.op(f"stablehlo.subtract {s2}, {y0}", th)
    mm = b.op(f"stablehlo.multiply %seven, {s3}", th)
    u = b.op(f"stablehlo.subtract {hz}, {mm}", th)
    hz2 = b.dus("%iterArg_2", u, ["%c_z", "%c_z"], t, th)
    body = "\n".join(b.lines)
    return f"""module @reactant_fdtd2d attributes {{mhlo.num_partitions = 1 : i64, mhlo.num_replicas = 1 : i64}} {{
  func.func @main(%arg0: {t} {{tf.aliasing_output = 0 : i32}}, %arg1: {t} {{tf.aliasing_output = 1 : i32}}, %arg2: {t} {{tf.aliasing_output = 2 : i32}}, %arg3: {tf}) -> ({t}, {t}, {t}) {{
    %c = stablehlo.constant dense<0> : tensor<i64>
    %c_0 = stablehlo.constant dense<{tmax}> : tensor<i64>
    %c_2 = stablehlo.constant dense<1> : tensor<i64>
    %c_1 = stablehlo.constant dense<1> : tensor<i32>
    %c_z = stablehlo.constant dense<0> : tensor<i32>
    %half_e = stablehlo.constant dense<5.000000e-01> : {te}
    %half_x = stablehlo.constant dense<5.000000e-01> : {tx}
    %seven = stablehlo.constant dense<0.699999988> : {th}
    %0:4 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0, %iterArg_1 = %arg1, %iterArg_2 = %arg2) : tensor<i64>, {t}, {t}, {t} attributes {{enzyme.disable_mincut}}
     cond {{
      %1 = stablehlo.compare  LT, %iterArg, %c_0 : (tensor<i64>, tensor<i64>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    }} do {{
      %1 = stablehlo.add %iterArg, %c_2 : tensor<i64>
{body}
      stablehlo.return %1, {ex2}, {ey2}, {hz2} : tensor<i64>, {t}, {t}, {t}
    }}
    return %0#1, %0#2, %0#3 : {t}, {t}, {t}
  }}
}}
"""


def jacobi1d(n: int, steps: int) -> str:
    """benchmark/polybench/stencil.jl:201-221 (jacobi_1d_vectorized): per iteration
    B[2:N-1] = (1/3) .* (A[1:N-2] .+ A[2:N-1] .+ A[3:N]), then the same from B into A."""
    t, ti = _t([n]), _t([n - 2])
    b = _Body()

    def half(src, dst):
        l, c, r = (b.slice(src, [(k, n - 2 + k)], t, ti) for k in range(3))
        s = b.op(f"stablehlo.add {l}, {c}", ti)
        s = b.op(f"stablehlo.add {s}, {r}", ti)
        u = b.op(f"stablehlo.multiply %third, {s}", ti)
        return b.dus(dst, u, ["%c_1"], t, ti)

    nb = half("%iterArg_0", "%iterArg_1")
    na = half(nb, "%iterArg_0")
    third = repr(float(__import__("numpy").float32(1.0 / 3.0)))
    return _two_array_loop("jacobi1d", [n], steps, [("%third", f"{float(third):.9e}", ti)], b.lines, na, nb)


def heat3d(n: int, steps: int) -> str:
    """benchmark/polybench/stencil.jl:125-169 (heat_3d_vectorized): per iteration the 7-point update
    0.125*(x[i+1] - 2x + x[i-1]) + 0.125*(x[j+1] - 2x + x[j-1]) + 0.125*(x[k+1] - 2x + x[k-1]) + x of the interior,
    from A into B and then from B into A.  Julia dim 1 (i) is the contiguous, i.e. last, tensor dim."""
    t, ti = _t([n, n, n]), _t([n - 2, n - 2, n - 2])
    b = _Body()
    m = n - 1

    def sl(src, dk, dj, di):  # offsets along Julia k, j, i = tensor dims 0, 1, 2
        return b.slice(src, [(1 + dk, m + dk), (1 + dj, m + dj), (1 + di, m + di)], t, ti)

    def half(src, dst):
        c = sl(src, 0, 0, 0)
        terms = []
        for axis in ("i", "j", "k"):
            d = {"i": (0, 0, 1), "j": (0, 1, 0), "k": (1, 0, 0)}[axis]
            hi = sl(src, *d)
            lo = sl(src, *(-x for x in d))
            two_c = b.op(f"stablehlo.multiply %two, {c}", ti)
            s = b.op(f"stablehlo.subtract {hi}, {two_c}", ti)
            s = b.op(f"stablehlo.add {s}, {lo}", ti)
            terms.append(b.op(f"stablehlo.multiply %eighth, {s}", ti))
        s = b.op(f"stablehlo.add {terms[0]}, {terms[1]}", ti)
        s = b.op(f"stablehlo.add {s}, {terms[2]}", ti)
        s = b.op(f"stablehlo.add {s}, {c}", ti)
        return b.dus(dst, s, ["%c_1", "%c_1", "%c_1"], t, ti)

    nb = half("%iterArg_0", "%iterArg_1")
    na = half(nb, "%iterArg_0")
    return _two_array_loop("heat3d", [n, n, n], steps, [("%two", "2.000000e+00", ti), ("%eighth", "1.250000e-01", ti)], b.lines, na, nb)
