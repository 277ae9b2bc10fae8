"""Randomly generated f32 fusion groups built only from exactly rounded operations: add, subtract, multiply,
divide, sqrt, min, max, abs, negate, floor, ceil, both roundings to integer, sign, clamp, comparisons in every
direction feeding selects, a round trip through bf16, and max / min reductions.  Each of these has one correctly
rounded f32 result (the oracle computes in f64 and rounds once, which gives the same value for these
operations), so both chain evaluators must equal the oracle exactly -- as values: the sign of a zero is not
compared, since minimum(-0, +0) may return either."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()

UNARY = ["negate", "abs", "floor", "ceil", "sign", "round_nearest_even", "round_nearest_afz"]
BINARY = ["add", "subtract", "multiply", "maximum", "minimum"]


def gen_case(seed):
    rng = np.random.default_rng(seed)
    rank = int(rng.integers(1, 4))
    dims = [int(rng.choice([1, 3, 8, 17, 64, 130])) for _ in range(rank)]
    if seed % 4 == 0:
        dims[-1] = int(rng.choice([256, 1024]))
    full = "x".join(map(str, dims))
    T, TI, TB = f"tensor<{full}xf32>", f"tensor<{full}xi1>", f"tensor<{full}xbf16>"
    args, inputs, lines, vals = [], [], [], []  # vals: (name, magnitude bound)

    def add_arg(shape):
        i = len(args)
        args.append(f"tensor<{'x'.join(map(str, shape))}xf32>")
        a = rng.uniform(-4.0, 4.0, size=shape).astype(np.float32)
        a[rng.random(size=shape) < 0.2] = np.float32(rng.choice([0.0, 0.5, -0.5, 1.5, -2.5, 3.0]))  # ties and zeros
        inputs.append(a)
        return f"%arg{i}"

    for _ in range(int(rng.integers(1, 4))):
        vals.append((add_arg(dims), 4.0))
    if rank >= 2 and rng.random() < 0.6:
        d = int(rng.integers(0, rank))
        a = add_arg([dims[d]])
        lines.append(f"    %bc = stablehlo.broadcast_in_dim {a}, dims = [{d}] : (tensor<{dims[d]}xf32>) -> {T}")
        vals.append(("%bc", 4.0))
    c = float(np.float32(rng.choice([0.25, 0.75, 1.5, 3.0])))
    lines.append(f"    %k = stablehlo.constant dense<{c!r}> : {T}")
    lines.append(f"    %lo = stablehlo.constant dense<-1.250000e+00> : {T}")
    vals.append(("%k", c))
    n_leaves = len(vals)
    n_ops = int(rng.integers(3, 14))
    pick = lambda: vals[-1] if rng.random() < 0.55 else vals[int(rng.integers(0, len(vals)))]
    for j in range(n_ops):
        name = f"%v{j}"
        r = rng.random()
        if r < 0.15:
            dirn = rng.choice(["GT", "LT", "GE", "LE", "EQ", "NE"])
            (x, bx), (y, by) = pick(), pick()
            lines.append(f"    %p{j} = stablehlo.compare {dirn}, {pick()[0]}, {pick()[0]} : ({T}, {T}) -> {TI}")
            lines.append(f"    {name} = stablehlo.select %p{j}, {x}, {y} : {TI}, {T}")
            vals.append((name, max(bx, by)))
        elif r < 0.27:  # divide by, or take the root of, something bounded away from zero
            (x, bx), (y, by) = pick(), pick()
            lines.append(f"    %g{j} = stablehlo.abs {y} : {T}")
            lines.append(f"    %h{j} = stablehlo.add %g{j}, %k : {T}")
            if rng.random() < 0.6:
                lines.append(f"    {name} = stablehlo.divide {x}, %h{j} : {T}")
                vals.append((name, bx / c))
            else:
                lines.append(f"    {name} = stablehlo.sqrt %h{j} : {T}")
                vals.append((name, float(np.sqrt(by + c))))
        elif r < 0.35:  # through bf16 and back
            x, bx = pick()
            lines.append(f"    %b{j} = stablehlo.convert {x} : ({T}) -> {TB}")
            lines.append(f"    {name} = stablehlo.convert %b{j} : ({TB}) -> {T}")
            vals.append((name, bx * 1.01))
        elif r < 0.42:
            x, bx = pick()
            lines.append(f"    {name} = stablehlo.clamp %lo, {x}, %k : {T}")
            vals.append((name, max(1.25, c)))
        elif r < 0.65:
            x, bx = pick()
            op = rng.choice(UNARY)
            lines.append(f"    {name} = stablehlo.{op} {x} : {T}")
            vals.append((name, 1.0 if op == "sign" else bx + 1.0))
        else:
            (x, bx), (y, by) = pick(), pick()
            ops = [o for o in BINARY if o != "multiply" or bx * by <= 1e6]
            op = rng.choice(ops)
            lines.append(f"    {name} = stablehlo.{op} {x}, {y} : {T}")
            vals.append((name, bx * by if op == "multiply" else (bx + by if op in ("add", "subtract") else max(bx, by))))
    last = vals[-1][0]
    results, rtypes = [], []
    mode = seed % 3
    if mode != 1:
        results.append(last); rtypes.append(T)
        mid = vals[n_leaves + n_ops // 2][0]
        if rng.random() < 0.4 and mid != last:
            results.append(mid); rtypes.append(T)
    if mode != 0:
        red_dims = sorted(rng.choice(rank, size=int(rng.integers(1, rank + 1)), replace=False).tolist())
        keep = [dims[d] for d in range(rank) if d not in red_dims]
        RT = f"tensor<{'x'.join(map(str, keep)) + 'x' if keep else ''}f32>"
        kind, init = [("maximum", "0xFF800000"), ("minimum", "0x7F800000")][int(rng.integers(0, 2))]
        lines.append(f"    %z = stablehlo.constant dense<{init}> : tensor<f32>")
        lines.append(f"    %red = stablehlo.reduce({last} init: %z) applies stablehlo.{kind} across dimensions = {red_dims} : ({T}, tensor<f32>) -> {RT}")
        results.append("%red"); rtypes.append(RT)
    lines.append(f"    return {', '.join(results)} : {', '.join(rtypes)}")
    sig = ", ".join(f"%arg{i}: {t}" for i, t in enumerate(args))
    text = f"module {{\n  func.func @main({sig}) -> ({', '.join(rtypes)}) {{\n" + "\n".join(lines) + "\n  }\n}\n"
    return text, inputs


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("RX_FUZZ_FIRST", "0")), int(os.environ.get("RX_FUZZ_FIRST", "0")) + int(os.environ.get("RX_FUZZ_CASES", "60"))))
def test_random_exactly_rounded_fusion_groups(seed):
    oracle, _ = entry.load_oracle()
    text, inputs = gen_case(seed)
    want = oracle.run_module(text, inputs)
    try:
        for threshold in (-1, 0):  # interpreter, then specialised kernels
            rx.chain_specialiser(threshold)
            f = rx.compile(text)
            r = f(*[rx.to_rarray(np.ascontiguousarray(a.T)) for a in inputs])
            r = r if isinstance(r, tuple) else (r,)
            for t, w in zip(r, want):
                got = np.ascontiguousarray(np.asarray(t).T)
                w = np.asarray(w, dtype=np.float32).reshape(got.shape)
                assert np.isfinite(w).all(), "the generator must not produce non-finite values"
                assert np.array_equal(got, w), f"threshold {threshold}, {int((got != w).sum())} elements differ\n{text}"
    finally:
        rx.chain_specialiser(1 << 20)
    assert rx.chain_specialiser_stats()["failed"] == 0
