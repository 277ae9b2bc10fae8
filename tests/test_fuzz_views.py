"""Randomly generated view chains: transposes, strided slices, reshapes and broadcasts composed in front of an
elementwise op and, sometimes, a reduction.  None of them may cost a pass over memory in the engine (they fold into
operand strides), and all of them must index exactly as the op definitions say (src/Ops.jl:761-793 slice, :1320-1357
broadcast_in_dim, :1273-1318 transpose / reshape): the map results are compared bit for bit with the numpy oracle."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()


def ty(shape, et="f32"):
    return "tensor<" + "".join(f"{d}x" for d in shape) + et + ">"


def gen_view_chain(rng, name, shape, lines, depth):
    """Applies `depth` random views to value `name` of `shape`; returns the new (name, shape)."""
    for k in range(depth):
        kind = rng.choice(["transpose", "slice", "reshape", "slice"])
        new = f"{name}_{k}"
        if kind == "transpose" and len(shape) >= 2:
            perm = rng.permutation(len(shape)).tolist()
            out = [shape[p] for p in perm]
            lines.append(f"    {new} = stablehlo.transpose {name}, dims = {perm} : ({ty(shape)}) -> {ty(out)}")
        elif kind == "slice":
            parts, out = [], []
            for d in shape:
                st = int(rng.integers(1, 3)) if d >= 6 and rng.random() < 0.4 else 1
                lo = int(rng.integers(0, max(1, d // 3)))
                hi = int(rng.integers(lo + 1, d + 1))
                n = (hi - lo + st - 1) // st
                parts.append(f"{lo}:{hi}" + (f":{st}" if st != 1 else ""))
                out.append(n)
            lines.append(f"    {new} = stablehlo.slice {name} [{', '.join(parts)}] : ({ty(shape)}) -> {ty(out)}")
        elif kind == "reshape" and len(shape) >= 2 and rng.random() < 0.5:
            i = int(rng.integers(0, len(shape) - 1))  # merge dims i, i+1
            out = shape[:i] + [shape[i] * shape[i + 1]] + shape[i + 2:]
            lines.append(f"    {new} = stablehlo.reshape {name} : ({ty(shape)}) -> {ty(out)}")
        elif kind == "reshape":
            i = int(rng.integers(0, len(shape)))  # split dim i by a divisor
            divs = [f for f in (2, 3, 4, 5) if shape[i] % f == 0 and shape[i] > f]
            if not divs or len(shape) >= 4:
                continue
            f = int(rng.choice(divs))
            out = shape[:i] + [f, shape[i] // f] + shape[i + 1:]
            lines.append(f"    {new} = stablehlo.reshape {name} : ({ty(shape)}) -> {ty(out)}")
        else:
            continue
        name, shape = new, list(out)
    return name, shape


def gen_case(seed):
    rng = np.random.default_rng(1000 + seed)
    rank = int(rng.integers(2, 4))
    shape = [int(rng.choice([4, 6, 8, 12, 20, 36])) for _ in range(rank)]
    lines = []
    a, ashape = gen_view_chain(rng, "%arg0", list(shape), lines, int(rng.integers(1, 5)))
    # second operand: a vector broadcast along a random dim of the viewed shape, or a full tensor of that shape
    inputs = [rng.standard_normal(shape).astype(np.float32)]
    args = [ty(shape)]
    if rng.random() < 0.6 and len(ashape) >= 1:
        d = int(rng.integers(0, len(ashape)))
        args.append(ty([ashape[d]]))
        inputs.append(rng.standard_normal([ashape[d]]).astype(np.float32))
        lines.append(f"    %b = stablehlo.broadcast_in_dim %arg1, dims = [{d}] : ({ty([ashape[d]])}) -> {ty(ashape)}")
    else:
        args.append(ty(ashape))
        inputs.append(rng.standard_normal(ashape).astype(np.float32))
        lines.append(f"    %b = stablehlo.transpose %arg1, dims = {list(range(len(ashape)))} : ({ty(ashape)}) -> {ty(ashape)}")
    op = rng.choice(["add", "multiply", "subtract", "maximum"])
    lines.append(f"    %r = stablehlo.{op} {a}, %b : {ty(ashape)}")
    results, rtypes = ["%r"], [ty(ashape)]
    if seed % 2 and len(ashape) >= 1:
        dims = sorted(rng.choice(len(ashape), size=int(rng.integers(1, len(ashape) + 1)), replace=False).tolist())
        keep = [ashape[d] for d in range(len(ashape)) if d not in dims]
        lines.append("    %z = stablehlo.constant dense<0.000000e+00> : tensor<f32>")
        lines.append(f"    %s = stablehlo.reduce(%r init: %z) applies stablehlo.add across dimensions = {dims} : ({ty(ashape)}, tensor<f32>) -> {ty(keep)}")
        results.append("%s"); rtypes.append(ty(keep))
    lines.append(f"    return {', '.join(results)} : {', '.join(rtypes)}")
    sig = ", ".join(f"%arg{i}: {t}" for i, t in enumerate(args))
    text = f"module {{\n  func.func @main({sig}) -> ({', '.join(rtypes)}) {{\n" + "\n".join(lines) + "\n  }\n}\n"
    return text, inputs, int(np.prod(ashape))


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("RX_FUZZ_FIRST", "0")), int(os.environ.get("RX_FUZZ_FIRST", "0")) + int(os.environ.get("RX_FUZZ_CASES", "60"))))
def test_random_view_chains(seed):
    oracle, _ = entry.load_oracle()
    text, inputs, n = gen_case(seed)
    want = oracle.run_module(text, inputs)
    f = rx.compile(text)
    r = f(*[rx.to_rarray(np.ascontiguousarray(a.T)) for a in inputs])
    r = r if isinstance(r, tuple) else (r,)
    got = [np.ascontiguousarray(np.asarray(t).T) for t in r]
    assert got[0].shape == tuple(np.asarray(want[0]).shape), text
    assert np.array_equal(got[0], np.asarray(want[0], dtype=np.float32)), text   # data movement + one exactly rounded op
    if len(got) > 1:
        tol = oracle.reduction_tolerance(max(n, 2)) * (np.abs(np.asarray(want[0], dtype=np.float64)).sum() + 1e-30)
        np.testing.assert_allclose(got[1], np.asarray(want[1], dtype=np.float64).reshape(got[1].shape), rtol=0, atol=tol, err_msg=text)
    if seed % 3 == 0:
        # the same program with every chain compiled at run time (the general map kernel then has the operands' strides
        # and the dims written into its source): the same bits as the interpreter kernels gave
        try:
            rx.chain_specialiser(0)
            r2 = rx.compile(text)(*[rx.to_rarray(np.ascontiguousarray(a.T)) for a in inputs])
        finally:
            rx.chain_specialiser(1 << 20)
        r2 = r2 if isinstance(r2, tuple) else (r2,)
        assert rx.chain_specialiser_stats()["failed"] == 0
        for a, b in zip(r, r2):
            assert np.asarray(a).tobytes() == np.asarray(b).tobytes(), text
