"""Randomly generated integer fusion groups: i32 arithmetic with wrap-around, bit operations, comparisons in every
direction feeding selects, iota, broadcast operands, a conversion to f32, and add / max / min reductions over any
subset of the dims.  Integer work has one right answer, so both chain evaluators (the on-GPU interpreter and the
run-time specialised kernels) must match the numpy oracle bit for bit."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()

UNARY = ["negate", "abs", "not"]
BINARY = ["add", "subtract", "multiply", "maximum", "minimum", "and", "or", "xor"]
EXTREMES = np.array([0, 1, -1, 2**31 - 1, -(2**31), 2**30, -(2**30) - 1, 65535, -65536], dtype=np.int64)


def gen_case(seed):
    rng = np.random.default_rng(seed)
    rank = int(rng.integers(1, 4))
    dims = [int(rng.choice([1, 2, 5, 16, 33, 128])) for _ in range(rank)]
    if seed % 4 == 0:
        dims[-1] = int(rng.choice([512, 2048]))
    full = "x".join(map(str, dims))
    T, TI, TF = f"tensor<{full}xi32>", f"tensor<{full}xi1>", f"tensor<{full}xf32>"
    args, inputs, lines, vals = [], [], [], []

    def add_arg(shape):
        i = len(args)
        args.append(f"tensor<{'x'.join(map(str, shape))}xi32>")
        a = rng.integers(-60, 60, size=shape, dtype=np.int64)
        wild = rng.random(size=shape) < 0.15  # a sprinkling of values that overflow under + and *
        a = np.where(wild, rng.choice(EXTREMES, size=shape), a).astype(np.int32)
        inputs.append(a)
        return f"%arg{i}"

    for _ in range(int(rng.integers(1, 4))):
        vals.append(add_arg(dims))
    if rank >= 2 and rng.random() < 0.6:
        d = int(rng.integers(0, rank))
        a = add_arg([dims[d]])
        lines.append(f"    %bc = stablehlo.broadcast_in_dim {a}, dims = [{d}] : (tensor<{dims[d]}xi32>) -> {T}")
        vals.append("%bc")
    if rng.random() < 0.6:
        d = int(rng.integers(0, rank))
        lines.append(f"    %io = stablehlo.iota dim = {d} : {T}")
        vals.append("%io")
    c = int(rng.choice([-7, -1, 2, 3, 255, 65537, 2**31 - 1]))
    lines.append(f"    %k = stablehlo.constant dense<{c}> : {T}")
    vals.append("%k")
    n_leaves = len(vals)
    n_ops = int(rng.integers(3, 14))
    pick = lambda: vals[-1] if rng.random() < 0.55 else vals[int(rng.integers(0, len(vals)))]
    for j in range(n_ops):
        name = f"%v{j}"
        r = rng.random()
        if r < 0.2:
            dirn = rng.choice(["GT", "LT", "GE", "LE", "EQ", "NE"])
            lines.append(f"    %p{j} = stablehlo.compare {dirn}, {pick()}, {pick()} : ({T}, {T}) -> {TI}")
            lines.append(f"    {name} = stablehlo.select %p{j}, {pick()}, {pick()} : {TI}, {T}")
        elif r < 0.4:
            lines.append(f"    {name} = stablehlo.{rng.choice(UNARY)} {pick()} : {T}")
        else:
            lines.append(f"    {name} = stablehlo.{rng.choice(BINARY)} {pick()}, {pick()} : {T}")
        vals.append(name)
    last = vals[-1]
    results, rtypes = [], []
    mode = seed % 3
    if mode != 1:
        if rng.random() < 0.3:  # leave the integers through an exact conversion
            lines.append(f"    %cf = stablehlo.convert {last} : ({T}) -> {TF}")
            results.append("%cf"); rtypes.append(TF)
        else:
            results.append(last); rtypes.append(T)
        mid = vals[n_leaves + n_ops // 2]
        if rng.random() < 0.4 and mid != last:
            results.append(mid); rtypes.append(T)
    if mode != 0:
        red_dims = sorted(rng.choice(rank, size=int(rng.integers(1, rank + 1)), replace=False).tolist())
        keep = [dims[d] for d in range(rank) if d not in red_dims]
        RT = f"tensor<{'x'.join(map(str, keep)) + 'x' if keep else ''}i32>"
        kind, init = [("add", "0"), ("maximum", str(-(2**31))), ("minimum", str(2**31 - 1))][int(rng.integers(0, 3))]
        lines.append(f"    %z = stablehlo.constant dense<{init}> : tensor<i32>")
        lines.append(f"    %red = stablehlo.reduce({last} init: %z) applies stablehlo.{kind} across dimensions = {red_dims} : ({T}, tensor<i32>) -> {RT}")
        results.append("%red"); rtypes.append(RT)
    lines.append(f"    return {', '.join(results)} : {', '.join(rtypes)}")
    sig = ", ".join(f"%arg{i}: {t}" for i, t in enumerate(args))
    text = f"module {{\n  func.func @main({sig}) -> ({', '.join(rtypes)}) {{\n" + "\n".join(lines) + "\n  }\n}\n"
    return text, inputs


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("RX_FUZZ_FIRST", "0")), int(os.environ.get("RX_FUZZ_FIRST", "0")) + int(os.environ.get("RX_FUZZ_CASES", "60"))))
def test_random_integer_fusion_groups(seed):
    oracle, _ = entry.load_oracle()
    text, inputs = gen_case(seed)
    with np.errstate(over="ignore"):
        want = oracle.run_module(text, inputs)
    try:
        for threshold in (-1, 0):  # interpreter, then specialised kernels
            rx.chain_specialiser(threshold)
            f = rx.compile(text)
            r = f(*[rx.to_rarray(np.ascontiguousarray(a.T)) for a in inputs])
            r = r if isinstance(r, tuple) else (r,)
            for t, w in zip(r, want):
                got = np.ascontiguousarray(np.asarray(t).T)
                w = np.asarray(w).reshape(got.shape)
                assert got.dtype == w.dtype, text
                assert np.array_equal(got.view(np.uint32), w.view(np.uint32)), f"threshold {threshold}\n{text}"
    finally:
        rx.chain_specialiser(1 << 20)
    assert rx.chain_specialiser_stats()["failed"] == 0
