"""Randomly generated fusion groups over a 1-D mesh of two devices: operands sharded along a random dimension (or
replicated when they do not vary along it), elementwise chains, and reductions that do or do not cross the sharded
dimension (local reduce + all-reduce, or a result that stays sharded).  Results must equal the unsharded numpy oracle
(src/xla/Sharding.jl:226-273 for the slicing rule; XLA's SPMD partitioner does this for the reference)."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()
NDEV = 2


def _ngpu():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def gen_case(seed):
    rng = np.random.default_rng(9000 + seed)
    dims = [int(rng.choice([2, 8, 34, 130])) * NDEV if k == 0 else int(rng.choice([1, 6, 64, 258])) * NDEV for k in range(2)]
    rng.shuffle(dims)
    dims = [int(d) for d in dims]
    s = int(rng.integers(0, 2))   # sharded boundary dim
    T = f"tensor<{dims[0]}x{dims[1]}xf32>"
    sh = lambda on: "{" + ('"x"' if on else "") + "}"
    full_attr = f' {{sdy.sharding = #sdy.sharding<@mesh, [{sh(s == 0)}, {sh(s == 1)}]>}}'
    args, inputs, specs, lines, vals = [], [], [], [], []
    for _ in range(2):
        args.append(f"%arg{len(args)}: {T}{full_attr}")
        inputs.append(rng.uniform(-1.5, 1.5, dims).astype(np.float32))
        specs.append("full")
        vals.append(f"%arg{len(args) - 1}")
    d = int(rng.integers(0, 2))
    vec_attr = f' {{sdy.sharding = #sdy.sharding<@mesh, [{sh(d == s)}]>}}'
    args.append(f"%arg2: tensor<{dims[d]}xf32>{vec_attr}")
    inputs.append(rng.uniform(-1.5, 1.5, [dims[d]]).astype(np.float32))
    specs.append("vec_sharded" if d == s else "vec_replicated")
    lines.append(f"    %bc = stablehlo.broadcast_in_dim %arg2, dims = [{d}] : (tensor<{dims[d]}xf32>) -> {T}")
    vals.append("%bc")
    lines.append(f"    %k = stablehlo.constant dense<7.500000e-01> : {T}")
    vals.append("%k")
    n_ops = int(rng.integers(3, 9))
    for j in range(n_ops):
        x = vals[-1] if rng.random() < 0.6 else vals[int(rng.integers(0, len(vals)))]
        y = vals[int(rng.integers(0, len(vals)))]
        if rng.random() < 0.4:
            op = rng.choice(["tanh", "sine", "abs", "negate", "logistic"])
            lines.append(f"    %v{j} = stablehlo.{op} {x} : {T}")
        else:
            op = rng.choice(["add", "subtract", "multiply", "maximum"])
            if op == "multiply":
                lines.append(f"    %t{j} = stablehlo.tanh {y} : {T}")
                y = f"%t{j}"
            lines.append(f"    %v{j} = stablehlo.{op} {x}, {y} : {T}")
        vals.append(f"%v{j}")
    last = vals[-1]
    results, rtypes, red_dims = [], [], None
    mode = seed % 3
    if mode != 1:
        results.append(last); rtypes.append(T)
    if mode != 0:
        red_dims = sorted(rng.choice(2, size=int(rng.integers(1, 3)), replace=False).tolist())
        keep = [dims[k] for k in range(2) if k not in red_dims]
        RT = f"tensor<{'x'.join(map(str, keep)) + 'x' if keep else ''}f32>"
        lines.append("    %z = stablehlo.constant dense<0.000000e+00> : tensor<f32>")
        lines.append(f"    %red = stablehlo.reduce({last} init: %z) applies stablehlo.add across dimensions = {red_dims} : ({T}, tensor<f32>) -> {RT}")
        results.append("%red"); rtypes.append(RT)
    lines.append(f"    return {', '.join(results)} : {', '.join(rtypes)}")
    text = (f'module attributes {{mhlo.num_partitions = {NDEV} : i64, mhlo.num_replicas = 1 : i64}} {{\n  sdy.mesh @mesh = <["x"={NDEV}]>\n'
            f"  func.func @main({', '.join(args)}) -> ({', '.join(rtypes)}) {{\n" + "\n".join(lines) + "\n  }\n}\n")
    plain = text.replace(full_attr, "").replace(vec_attr, "").replace(f"mhlo.num_partitions = {NDEV}", "mhlo.num_partitions = 1")
    plain = "\n".join(l for l in plain.splitlines() if "sdy.mesh" not in l) + "\n"
    return text, plain, inputs, specs, dims, s, d, red_dims, n_ops


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("RX_FUZZ_FIRST", "0")), int(os.environ.get("RX_FUZZ_FIRST", "0")) + int(os.environ.get("RX_FUZZ_CASES", "40"))))
def test_random_sharded_fusion_groups(seed):
    if _ngpu() < NDEV:
        pytest.skip("needs 2 GPUs")
    oracle, _ = entry.load_oracle()
    text, plain, inputs, specs, dims, s, d, red_dims, n_ops = gen_case(seed)
    want = oracle.run_module(plain, inputs)
    client = rx.Client(allowed_devices=list(range(NDEV)))
    try:
        mesh = rx.Mesh(client.devices, ("x",))
        # host arrays are column-major: boundary dim k of a rank-2 array is host dim 1 - k
        full = rx.NamedSharding(mesh, tuple("x" if (1 - k) == s else None for k in range(2)))
        up = []
        for a, spec in zip(inputs, specs):
            if spec == "full":
                up.append(rx.to_rarray(np.ascontiguousarray(a.T), client, sharding=full))
            elif spec == "vec_sharded":
                up.append(rx.to_rarray(a, client, sharding=rx.NamedSharding(mesh, ("x",))))
            else:
                up.append(rx.to_rarray(a, client, sharding=rx.NamedSharding(mesh, (None,))))
        r = rx.compile(text, client)(*up)
        r = r if isinstance(r, tuple) else (r,)
        got = [np.asarray(t) for t in r]
    finally:
        client.close()
    for g, w in zip(got, want):
        w = np.asarray(w, dtype=np.float64)
        g = g.T if g.ndim == 2 else g
        assert g.shape == w.shape, (g.shape, w.shape, text)
        n = 1 if g.ndim == 2 else int(np.prod([dims[k] for k in red_dims]))
        scale = 8.0
        tol = 4e-7 * (n_ops + 4) * scale * n + (oracle.reduction_tolerance(max(n, 2)) * scale * n if n > 1 else 0)
        np.testing.assert_allclose(g, w, rtol=0, atol=tol, err_msg=text)
