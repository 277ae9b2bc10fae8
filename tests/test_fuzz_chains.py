"""Randomly generated fusion groups: elementwise DAGs over broadcast operands, optionally reduced, run through the
engine with the on-GPU interpreter and with run-time specialised kernels.  The two evaluators must agree bit for
bit; both must agree with the numpy oracle within a bound derived from the magnitudes in the program.  The
generator only emits ops where a last-bit difference in libm cannot flip a branch (comparisons are made on
inputs, which are exact), so the tolerance stays tight."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()

UNARY = {  # op -> (bound of the result given bound b of the operand, allowed if)
    "sine": (lambda b: 1.0, lambda b: b <= 50),
    "cosine": (lambda b: 1.0, lambda b: b <= 50),
    "tanh": (lambda b: 1.0, lambda b: True),
    "negate": (lambda b: b, lambda b: True),
    "abs": (lambda b: b, lambda b: True),
    "logistic": (lambda b: 1.0, lambda b: b <= 30),
    "exponential": (lambda b: float(np.exp(b)), lambda b: b <= 3),
}
BINARY = {
    "add": (lambda a, b: a + b, lambda a, b: True),
    "subtract": (lambda a, b: a + b, lambda a, b: True),
    "multiply": (lambda a, b: a * b, lambda a, b: a * b <= 1e3),
    "maximum": (lambda a, b: max(a, b), lambda a, b: True),
    "minimum": (lambda a, b: max(a, b), lambda a, b: True),
}


def gen_case(seed):
    rng = np.random.default_rng(seed)
    rank = int(rng.integers(1, 4))
    dims = [int(rng.choice([1, 3, 8, 17, 64, 130])) for _ in range(rank)]
    if seed % 5 == 0:
        dims[-1] = int(rng.choice([256, 1024]))  # wide enough for the vector paths
    full = "x".join(map(str, dims))
    T = f"tensor<{full}xf32>"
    TI = f"tensor<{full}xi1>"
    args, inputs, lines, vals = [], [], [], []  # vals: (name, bound)

    def add_arg(shape, dt="f32"):
        i = len(args)
        ts = "x".join(map(str, shape))
        args.append(f"tensor<{ts + 'x' if ts else ''}{dt}>")
        a = rng.uniform(-1.5, 1.5, size=shape).astype(np.float32)
        if dt == "bf16":
            a = a.astype(rx.bfloat16)
        inputs.append(a)
        return f"%arg{i}"

    # full-shape f32 operands
    for _ in range(int(rng.integers(2, 4))):
        vals.append((add_arg(dims), 1.5))
    # a bf16 operand converted on the way in
    if rng.random() < 0.4:
        a = add_arg(dims, "bf16")
        lines.append(f"    %cv = stablehlo.convert {a} : (tensor<{full}xbf16>) -> {T}")
        vals.append(("%cv", 1.5))
    # a vector broadcast along one dim
    if rank >= 2 and rng.random() < 0.7:
        d = int(rng.integers(0, rank))
        a = add_arg([dims[d]])
        lines.append(f"    %bc = stablehlo.broadcast_in_dim {a}, dims = [{d}] : (tensor<{dims[d]}xf32>) -> {T}")
        vals.append(("%bc", 1.5))
    # a splat constant
    c = float(np.float32(rng.uniform(0.25, 2.0)))
    lines.append(f"    %k = stablehlo.constant dense<{c!r}> : {T}")
    vals.append(("%k", c))
    leaves = list(vals)
    n_ops = int(rng.integers(4, 15))
    for j in range(n_ops):
        name = f"%v{j}"
        pick = lambda: vals[-1] if rng.random() < 0.6 else vals[int(rng.integers(0, len(vals)))]
        r = rng.random()
        if r < 0.08 and len(leaves) >= 2:  # select on a comparison of two inputs
            (la, _), (lb, _) = leaves[int(rng.integers(0, len(leaves)))], leaves[int(rng.integers(0, len(leaves)))]
            (x, bx), (y, by) = pick(), pick()
            dirn = rng.choice(["GT", "LT", "GE", "LE"])
            lines.append(f"    %p{j} = stablehlo.compare {dirn}, {la}, {lb} : ({T}, {T}) -> {TI}")
            lines.append(f"    {name} = stablehlo.select %p{j}, {x}, {y} : {TI}, {T}")
            vals.append((name, max(bx, by)))
        elif r < 0.16:  # guarded divide / sqrt / log
            (x, bx), (y, by) = pick(), pick()
            lines.append(f"    %g{j} = stablehlo.abs {y} : {T}")
            lines.append(f"    %h{j} = stablehlo.add %g{j}, %k : {T}")
            kind = rng.choice(["divide", "sqrt", "log", "rsqrt"])
            if kind == "divide":
                lines.append(f"    {name} = stablehlo.divide {x}, %h{j} : {T}")
                vals.append((name, bx / c))
            else:
                lines.append(f"    {name} = stablehlo.{kind} %h{j} : {T}")
                vals.append((name, max(abs(np.log(c)), np.log(by + c), np.sqrt(by + c), 1 / np.sqrt(c))))
        elif r < 0.5:
            ops = [o for o in UNARY if UNARY[o][1](pick()[1])]
            x, bx = pick()
            ops = [o for o in UNARY if UNARY[o][1](bx)]
            op = rng.choice(ops)
            lines.append(f"    {name} = stablehlo.{op} {x} : {T}")
            vals.append((name, UNARY[op][0](bx)))
        else:
            (x, bx), (y, by) = pick(), pick()
            ops = [o for o in BINARY if BINARY[o][1](bx, by)]
            op = rng.choice(ops)
            lines.append(f"    {name} = stablehlo.{op} {x}, {y} : {T}")
            vals.append((name, BINARY[op][0](bx, by)))
    scale = max(b for _, b in vals)
    results, rtypes, kinds = [], [], []
    last = vals[-1][0]
    mode = seed % 3
    if mode != 1:
        results.append(last); rtypes.append(T); kinds.append(("map", 1))
        if rng.random() < 0.4:  # a second output from the middle of the chain
            mid = vals[len(leaves) + n_ops // 2][0] if len(vals) > len(leaves) + n_ops // 2 else last
            if mid != last and mid.startswith("%v"):
                results.append(mid); rtypes.append(T); kinds.append(("map", 1))
    if mode != 0:
        red_dims = sorted(rng.choice(rank, size=int(rng.integers(1, rank + 1)), replace=False).tolist())
        keep = [dims[d] for d in range(rank) if d not in red_dims]
        RT = f"tensor<{'x'.join(map(str, keep)) + 'x' if keep else ''}f32>"
        kind = "add" if rng.random() < 0.7 else "maximum"
        init = "0.000000e+00" if kind == "add" else "0xFF800000"
        lines.append(f"    %z = stablehlo.constant dense<{init}> : tensor<f32>")
        lines.append(f"    %red = stablehlo.reduce({last} init: %z) applies stablehlo.{kind} across dimensions = {red_dims} : ({T}, tensor<f32>) -> {RT}")
        n_red = int(np.prod([dims[d] for d in red_dims]))
        results.append("%red"); rtypes.append(RT); kinds.append((kind, n_red))
    lines.append(f"    return {', '.join(results)} : {', '.join(rtypes)}")
    sig = ", ".join(f"%arg{i}: {t}" for i, t in enumerate(args))
    text = f"module {{\n  func.func @main({sig}) -> ({', '.join(rtypes)}) {{\n" + "\n".join(lines) + "\n  }\n}\n"
    return text, inputs, kinds, scale, n_ops


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("RX_FUZZ_FIRST", "0")), int(os.environ.get("RX_FUZZ_FIRST", "0")) + int(os.environ.get("RX_FUZZ_CASES", "60"))))
def test_random_fusion_groups(seed):
    oracle, _ = entry.load_oracle()
    text, inputs, kinds, scale, n_ops = gen_case(seed)
    want = oracle.run_module(text, inputs)
    outs = {}
    try:
        for mode, threshold in (("interpreter", -1), ("specialised", 0)):
            rx.chain_specialiser(threshold)
            f = rx.compile(text)
            r = f(*[rx.to_rarray(np.ascontiguousarray(a.T)) for a in inputs])
            r = r if isinstance(r, tuple) else (r,)
            outs[mode] = [np.ascontiguousarray(np.asarray(t).T) for t in r]
    finally:
        rx.chain_specialiser(1 << 20)
    assert rx.chain_specialiser_stats()["failed"] == 0
    for a, b in zip(outs["interpreter"], outs["specialised"]):
        assert a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32)), text
    for got, w, (kind, n) in zip(outs["specialised"], want, kinds):
        w = np.asarray(w, dtype=np.float64).reshape(got.shape)
        # each op contributes a few ulp of its operands' magnitude; sums of n terms add the reduction bound
        tol = 4e-7 * (n_ops + 4) * scale
        if kind == "add":
            tol = tol * n + oracle.reduction_tolerance(max(n, 2)) * scale * n
        np.testing.assert_allclose(got, w, rtol=0, atol=tol, err_msg=text)


def to_f64(text, inputs):
    """The same random program on Float64 arrays (bf16 operands stay bf16 and are widened by their convert)."""
    t = text.replace("xf32>", "xf64>").replace("tensor<f32>", "tensor<f64>").replace("0xFF800000", "0xFFF0000000000000")
    ins = [a if a.dtype == rx.bfloat16 else a.astype(np.float64) for a in inputs]
    return t, ins


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("RX_FUZZ_FIRST", "0")), int(os.environ.get("RX_FUZZ_FIRST", "0")) + int(os.environ.get("RX_FUZZ_CASES", "60"))))
def test_random_fusion_groups_in_float64(seed):
    """Wide programs (64-bit registers, the interpreter kernels of rx_wide.cu) against the oracle, which evaluates
    f64 modules in float64: a few ulp of double per op."""
    oracle, _ = entry.load_oracle()
    text, inputs, kinds, scale, n_ops = gen_case(seed)
    text, inputs = to_f64(text, inputs)
    want = oracle.run_module(text, inputs)
    f = rx.compile(text)
    r = f(*[rx.to_rarray(np.ascontiguousarray(a.T)) for a in inputs])
    r = r if isinstance(r, tuple) else (r,)
    outs = [np.ascontiguousarray(np.asarray(t).T) for t in r]
    for got, w, (kind, n) in zip(outs, want, kinds):
        assert got.dtype == np.float64
        w = np.asarray(w, dtype=np.float64).reshape(got.shape)
        tol = 1e-15 * (n_ops + 4) * scale * 4
        if kind == "add":
            tol = tol * n + 1e-15 * scale * n * np.sqrt(max(n, 2))
        np.testing.assert_allclose(got, w, rtol=0, atol=tol, err_msg=text)
