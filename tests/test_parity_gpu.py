"""Parity of the CUDA path with the CPU oracle, through the C ABI (ctypes).

Bars (from the benchmark contract): bit-exact for indexing / slicing / integer
work; fp32 reductions within 1e-5*sqrt(log2 n) relative to the float64 result
(relative to the 2-norm of the terms where the sum itself is ill-conditioned);
bf16 dot_general within 2e-2 of the fp32 result.
"""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
NP = {"f64": np.float64, "f32": np.float32, "i32": np.int32, "i1": np.bool_}


def run(rx, client, text, inputs_xla, **kw):
    """inputs in the boundary layout (row-major over the tensor dims)."""
    f = rx.compile(text, client)
    args = [rx.to_rarray(np.asarray(a).T, client) for a in inputs_xla]
    out = f(*args, **kw)
    outs = out if isinstance(out, tuple) else (out,)
    return [np.asarray(o).T for o in outs], f, args


# ---------------------------------------------------------------- sinsum (C1)
@pytest.mark.parametrize("n", [1, 3, 127, 4096, (1 << 20) + 1, 1 << 24])
@pytest.mark.parametrize("raw", [False, True])
def test_sinsum_add(rx, ref, client, n, raw):
    rng = np.random.default_rng(n)
    x = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
    y = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
    text = rx.programs.sinsum_add(n, raw=raw)
    (got,), f, args = run(rx, client, text, [x, y])
    terms = np.sin(x.astype(np.float64)) + y.astype(np.float64)
    want = terms.sum()
    tol = ref.reduction_tolerance(n)
    assert abs(float(got) - want) <= tol * max(abs(want), np.linalg.norm(terms)), (float(got), want)
    # deterministic two-pass combine: same bits on a second run
    again = np.asarray(f(*args)).T
    assert again.tobytes() == np.asarray(got).tobytes()


def test_sinsum_large_arguments_take_the_slow_range_reduction(rx, ref, client):
    n = 10007
    rng = np.random.default_rng(5)
    x = (rng.uniform(-1, 1, n) * 1e6).astype(np.float32)
    y = np.zeros(n, np.float32)
    (got,), _, _ = run(rx, client, rx.programs.sinsum_add(n), [x, y])
    terms = np.sin(x.astype(np.float64))
    assert abs(float(got) - terms.sum()) <= 1e-5 * np.linalg.norm(terms) * 4


# ---------------------------------------------------------------- generic chains
def module(args, results, body):
    a = ", ".join(f"%arg{i}: {t}" for i, t in enumerate(args))
    return f"module {{\n  func.func @main({a}) -> ({', '.join(results)}) {{\n{body}\n  }}\n}}\n"


def test_generic_map_chain(rx, ref, client):
    n = 100003
    t = f"tensor<{n}xf32>"
    text = module([t, t], [t], f"""    %c = stablehlo.constant dense<2.500000e+00> : {t}
    %0 = stablehlo.tanh %arg0 : {t}
    %1 = stablehlo.multiply %0, %arg1 : {t}
    %2 = stablehlo.add %1, %c : {t}
    %3 = stablehlo.exponential %arg1 : {t}
    %4 = stablehlo.maximum %2, %3 : {t}
    %5 = stablehlo.compare  GT, %arg0, %arg1 : ({t}, {t}) -> tensor<{n}xi1>
    %6 = stablehlo.select %5, %4, %arg0 : tensor<{n}xi1>, {t}
    return %6 : {t}""")
    rng = np.random.default_rng(7)
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    (got,), _, _ = run(rx, client, text, [x, y])
    want = ref.run_module(text, [x, y])[0]
    np.testing.assert_allclose(got, want, rtol=4e-6, atol=1e-7)


def test_generic_reduce_chain_and_strided_operands(rx, ref, client):
    # sum(x .* x') : one operand is read transposed
    t = "tensor<37x37xf32>"
    text = module([t], ["tensor<f32>"], f"""    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %0 = stablehlo.transpose %arg0, dims = [1, 0] : ({t}) -> {t}
    %1 = stablehlo.multiply %arg0, %0 : {t}
    %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [0, 1] : ({t}, tensor<f32>) -> tensor<f32>
    return %2 : tensor<f32>""")
    x = np.random.default_rng(8).standard_normal((37, 37)).astype(np.float32)
    (got,), _, _ = run(rx, client, text, [x])
    want = ref.run_module(text, [x])[0]
    np.testing.assert_allclose(got, want, rtol=2e-5)


@pytest.mark.parametrize("dims,keep", [([1], "96x40"), ([0], "64x40"), ([2], "96x64"), ([0, 1], "40"), ([1, 2], "96"), ([0, 1, 2], "")])
@pytest.mark.parametrize("kind,init", [("add", "0.000000e+00"), ("maximum", "0xFF800000")])
def test_axis_reductions(rx, ref, client, dims, keep, kind, init):
    t = "tensor<96x64x40xf32>"
    tr = f"tensor<{keep + 'x' if keep else ''}f32>"
    text = module([t], [tr], f"""    %cst = stablehlo.constant dense<{init}> : tensor<f32>
    %0 = stablehlo.cosine %arg0 : {t}
    %1 = stablehlo.reduce(%0 init: %cst) applies stablehlo.{kind} across dimensions = {dims} : ({t}, tensor<f32>) -> {tr}
    return %1 : {tr}""")
    x = np.random.default_rng(9).standard_normal((96, 64, 40)).astype(np.float32)
    (got,), _, _ = run(rx, client, text, [x])
    want = ref.run_module(text, [x])[0]
    np.testing.assert_allclose(got, want, rtol=3e-5, atol=3e-5)


with open(os.path.join(HERE, "golden", "reactant_fixtures.json")) as f:
    CASES = [c for c in json.load(f)["cases"] if c["element_type"] != "f64" and "sharded" not in c["name"]]


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_reference_fixtures_through_the_engine(rx, ref, client, case):
    mod = ref.parse_module(case["module"])
    ins = [np.array(s["data"], dtype=NP[et]).reshape(s["dims"]) for (_, (_, et)), s in zip(mod["funcs"]["main"].args, case["inputs"])]
    got, _, _ = run(rx, client, case["module"], ins)
    for g, e in zip(got, case["expected"]):
        want = np.array(e["data"], dtype=np.float64).reshape(e["dims"])
        assert list(g.shape) == e["dims"]
        if case["rtol"] == 0.0:
            assert np.array_equal(g, want.astype(g.dtype))
        else:
            np.testing.assert_allclose(g.astype(np.float64), want, rtol=max(case["rtol"], 4e-6))


# ---------------------------------------------------------------- logsumexp (C2)
@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 3), (1000, 17), (4096, 8), (2049, 5), (32768, 64)])
@pytest.mark.parametrize("raw", [False, True])
def test_logsumexp_dims1(rx, ref, client, rows, cols, raw):
    x = np.random.default_rng(rows * 31 + cols).standard_normal((cols, rows)).astype(np.float32)
    text = rx.programs.logsumexp_dims1(rows, cols, raw=raw)
    (got,), f, _ = run(rx, client, text, [x])
    if rows > 1 and cols > 1:  # degenerate shapes collapse to plain maps
        assert [s["kind"] for s in f.describe()["steps"]] == ["logsumexp"]
    want = ref.run_module(text, [x])[0]
    assert got.shape == want.shape == (cols, 1)
    np.testing.assert_allclose(got, want, rtol=ref.reduction_tolerance(rows))


def test_logsumexp_with_infinities(rx, ref, client):
    rows, cols = 300, 4
    x = np.random.default_rng(2).standard_normal((cols, rows)).astype(np.float32)
    x[0, 5] = -np.inf
    x[1, :] = -np.inf
    x[1, 7] = 1.5
    x[2, 9] = 80.0
    x[3, 0] = np.inf
    text = rx.programs.logsumexp_dims1(rows, cols)
    (got,), _, _ = run(rx, client, text, [x])
    with np.errstate(all="ignore"):
        want = ref.run_module(text, [x])[0]
    np.testing.assert_allclose(got[:3], want[:3], rtol=1e-5)
    assert np.isnan(got[3, 0]) and np.isnan(want[3, 0])  # inf - inf inside the op sequence


def test_logsumexp_full_size_against_c_oracle(rx, ref, cpu, client):
    rows, cols = 32768, 8192
    x = np.random.default_rng(3).standard_normal((cols, rows), dtype=np.float32)
    (got,), _, _ = run(rx, client, rx.programs.logsumexp_dims1(rows, cols), [x])
    want = cpu.logsumexp_dims1(x)
    np.testing.assert_allclose(got.reshape(-1), want, rtol=ref.reduction_tolerance(rows))
    # shift invariance: logsumexp(x + c) = logsumexp(x) + c
    (got2,), _, _ = run(rx, client, rx.programs.logsumexp_dims1(rows, 64), [x[:64] + np.float32(3.0)])
    np.testing.assert_allclose(got2.reshape(-1), want[:64] + 3.0, rtol=1e-5)


# ---------------------------------------------------------------- Jacobi-2D (C3)
@pytest.mark.parametrize("n,steps", [(3, 1), (4, 3), (8, 2), (33, 5), (130, 4), (515, 3), (1030, 2)])
@pytest.mark.parametrize("form", ["dus", "pad", "concat"])
def test_jacobi2d_bit_exact(rx, ref, client, n, steps, form):
    rng = np.random.default_rng(n)
    a = rng.random((n, n), dtype=np.float32)
    b = rng.random((n, n), dtype=np.float32)
    text = rx.programs.jacobi2d(n, steps, form=form)
    (ga, gb), _, _ = run(rx, client, text, [a, b])
    wa, wb = ref.run_module(text, [a, b])
    assert np.array_equal(ga, wa) and np.array_equal(gb, wb)


@pytest.mark.parametrize("n", [1028, 516, 2052])
@pytest.mark.parametrize("steps", [2, 3, 4, 5, 7, 12])
def test_counted_stencil_loop_is_one_launch_and_bit_exact(rx, ref, client, steps, n):
    """A loop whose body is only 5-point updates runs as one cooperative launch with grid barriers between the
    sweeps; an odd trip count leaves the arrays swapped exactly as sweep-by-sweep execution does.  From four sweeps
    on, all but the last two (three, for an odd count) are done two per pass over memory, through a scratch array:
    same bits, and both carried arrays end with what the one-sweep-at-a-time loop leaves.  (The row pitch must be a
    multiple of 16 bytes for the TMA path; other sizes run the strided map kernel sweep by sweep.)"""
    rng = np.random.default_rng(steps)
    a = rng.random((n, n), dtype=np.float32)
    b = rng.random((n, n), dtype=np.float32)
    text = rx.programs.jacobi2d(n, steps)
    dev = client.addressable_devices[0]
    f = rx.compile(text, client)
    A, B = rx.to_rarray(a.T, client), rx.to_rarray(b.T, client)
    before = dev.kernel_launches()
    out = f(A, B)
    assert dev.kernel_launches() - before == 1
    ga, gb = [np.asarray(o).T for o in out]
    wa, wb = ref.run_module(text, [a, b])
    assert np.array_equal(ga, wa) and np.array_equal(gb, wb)


@pytest.mark.parametrize("steps", [1, 2, 3, 6])
def test_two_half_step_loop_is_one_launch_and_bit_exact(rx, ref, client, steps, monkeypatch):
    """The reference's own spelling (two updates per iteration, no swap; a different order of the additions): also one
    launch, also two sweeps per pass from four sweeps on, and the same bits with that turned off."""
    n = 1028
    rng = np.random.default_rng(steps)
    a = rng.random((n, n), dtype=np.float32)
    b = rng.random((n, n), dtype=np.float32)
    text = rx.programs.jacobi2d(n, steps, form="halfsteps")
    dev = client.addressable_devices[0]
    f = rx.compile(text, client)
    before = dev.kernel_launches()
    out = f(rx.to_rarray(a.T, client), rx.to_rarray(b.T, client))
    assert dev.kernel_launches() - before == (1 if steps >= 2 else 2)   # a single iteration is not worth a cooperative launch
    ga, gb = [np.asarray(o).T for o in out]
    wa, wb = ref.run_module(text, [a, b])
    assert np.array_equal(ga, wa) and np.array_equal(gb, wb)
    monkeypatch.setenv("RX_STENCIL_FUSE2", "0")
    out = f(rx.to_rarray(a.T, client), rx.to_rarray(b.T, client))
    assert all(np.array_equal(np.asarray(o).T, w) for o, w in zip(out, (wa, wb)))
    # tiles handed out in a fixed pattern instead of from the per-pass queue: with and without double sweeps
    monkeypatch.setenv("RX_STENCIL_QUEUE", "0")
    out = f(rx.to_rarray(a.T, client), rx.to_rarray(b.T, client))
    assert all(np.array_equal(np.asarray(o).T, w) for o, w in zip(out, (wa, wb)))
    monkeypatch.delenv("RX_STENCIL_FUSE2")
    out = f(rx.to_rarray(a.T, client), rx.to_rarray(b.T, client))
    assert all(np.array_equal(np.asarray(o).T, w) for o, w in zip(out, (wa, wb)))


def test_jacobi2d_full_size_against_c_oracle(rx, cpu, client):
    n, steps = 8192, 4
    rng = np.random.default_rng(4)
    a = rng.random((n, n), dtype=np.float32)
    b = rng.random((n, n), dtype=np.float32)
    (ga, gb), _, _ = run(rx, client, rx.programs.jacobi2d(n, steps), [a, b])
    wa, wb = cpu.jacobi2d(a, b, steps)
    assert np.array_equal(ga, wa) and np.array_equal(gb, wb)
    # boundary rows/cols of both arrays are never written
    assert np.array_equal(ga[0], a[0] if steps % 2 == 0 else b[0])


def test_donated_arguments_follow_their_results(rx, ref, client):
    n = 64
    a = np.random.default_rng(1).random((n, n), dtype=np.float32)
    b = np.zeros((n, n), np.float32)
    text = rx.programs.jacobi2d(n, 1)
    f = rx.compile(text, client)
    A, B = rx.to_rarray(a.T, client), rx.to_rarray(b.T, client)
    old_a = A.data[0]
    ra, rb = f(A, B)
    wa, wb = ref.run_module(text, [a, b])
    assert np.array_equal(np.asarray(A).T, wa) and np.array_equal(np.asarray(B).T, wb)
    with pytest.raises(rx.ReactantError) as e:  # the donated handle is dead
        old_a.to_host()
    assert e.value.code == 7
    # without donation the inputs stay intact and the results are fresh
    A2, B2 = rx.to_rarray(a.T, client), rx.to_rarray(b.T, client)
    ra2, rb2 = f(A2, B2, donate=False)
    assert np.array_equal(np.asarray(A2).T, a) and np.array_equal(np.asarray(B2).T, b)
    assert np.array_equal(np.asarray(ra2).T, wa) and np.array_equal(np.asarray(rb2).T, wb)


# ---------------------------------------------------------------- dot_general (C4)
@pytest.mark.parametrize("m,k,n", [(50, 70, 30), (128, 256, 128), (257, 129, 65)])
def test_matmul_f32(rx, ref, client, m, k, n):
    rng = np.random.default_rng(m)
    a = rng.standard_normal((k, m)).astype(np.float32)
    b = rng.standard_normal((n, k)).astype(np.float32)
    text = rx.programs.matmul(m, k, n)
    (got,), _, _ = run(rx, client, text, [a, b])
    want = ref.run_module(text, [a, b])[0]
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (256, 512, 384), (1024, 1024, 512), (200, 72, 136), (520, 200, 392), (2048, 4096, 1024)])
def test_matmul_bf16(rx, ref, client, m, k, n):
    rng = np.random.default_rng(k)
    a = ref.round_to_bf16(rng.standard_normal((k, m)).astype(np.float32))
    b = ref.round_to_bf16(rng.standard_normal((n, k)).astype(np.float32))
    text = rx.programs.matmul(m, k, n, et="bf16")
    f = rx.compile(text, client)
    out = f(rx.to_rarray(a.T.astype(rx.bfloat16), client), rx.to_rarray(b.T.astype(rx.bfloat16), client))
    got = np.asarray(out).T.astype(np.float32)
    want = b.astype(np.float64) @ a.astype(np.float64)
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err <= 2e-2, err
    # tighter: only the final bf16 rounding separates us from the fp32 result
    np.testing.assert_allclose(got, want, rtol=2 ** -7, atol=np.abs(want).max() * 2 ** -8)


def test_native_kernel_families_are_the_ones_that_run(rx, ref, client):
    """bf16 contractions must run on the tcgen05 kernel and stencil steps on the TMA kernel
    (the CUDA-core / generic kernels exist only for shapes those cannot take)."""
    dev = client.addressable_devices[0]
    dev.profile()
    dev.set_profiling(True)
    try:
        a = np.ones((256, 128), np.float32).astype(rx.bfloat16)
        f = rx.compile(rx.programs.matmul(128, 256, 256, et="bf16"), client)
        f(rx.to_rarray(a.T, client), rx.to_rarray(np.ones((256, 256), np.float32).astype(rx.bfloat16), client))
        g = rx.compile(rx.programs.jacobi2d(300, 2), client)
        z = np.zeros((300, 300), np.float32)
        g(rx.to_rarray(z, client), rx.to_rarray(z, client))
        dev.synchronize()
    finally:
        dev.set_profiling(False)
    prof = dev.profile()
    assert prof.get("gemm_tc", {}).get("launches") == 1 and "gemm_simt" not in prof, prof
    # both sweeps of the counted loop in one cooperative launch of the TMA kernel
    assert prof.get("stencil_tma_loop", {}).get("launches") == 1 and "stencil_generic" not in prof and "stencil_tma" not in prof, prof


def mlp_inputs(ref, F, H, O, B, seed=6):
    rng = np.random.default_rng(seed)
    bf = lambda a: ref.round_to_bf16(a.astype(np.float32))
    X = bf(rng.standard_normal((B, F)))
    W1 = bf(rng.standard_normal((F, H)) / np.sqrt(F))
    W2 = bf(rng.standard_normal((H, O)) / np.sqrt(H))
    b1 = (0.01 * rng.standard_normal(H)).astype(np.float32)
    b2 = (0.01 * rng.standard_normal(O)).astype(np.float32)
    Y = rng.standard_normal((B, O)).astype(np.float32)
    return [W1, b1, W2, b2, X, Y]


@pytest.mark.parametrize("F,H,O,B", [(64, 128, 32, 256), (128, 256, 128, 128), (256, 512, 256, 512), (320, 768, 264, 384)])
def test_mlp_forward_and_gradients(rx, ref, client, F, H, O, B):
    ins = mlp_inputs(ref, F, H, O, B)
    text = rx.programs.mlp_grad(F, H, O, B)
    f = rx.compile(text, client)
    conv = lambda a: a.T.astype(rx.bfloat16) if a.ndim == 2 and a is not ins[5] else a.T
    outs = f(*[rx.to_rarray(conv(a), client) for a in ins])
    got = [np.asarray(o).T.astype(np.float32) for o in outs]
    want = ref.run_module(text, ins)
    for name, g, w in zip(("dW1", "db1", "dW2", "db2", "loss"), got, want):
        scale = np.abs(w).max()
        assert np.abs(g - w).max() <= 2e-2 * scale, (name, np.abs(g - w).max(), scale)


# ---------------------------------------------------------------- boundary errors
def test_shape_mismatch_and_bad_arity_are_errors(rx, client):
    f = rx.compile(rx.programs.sinsum_add(16), client)
    x = rx.to_rarray(np.zeros(16, np.float32), client)
    y = rx.to_rarray(np.zeros(8, np.float32), client)
    with pytest.raises(rx.ReactantError) as e:
        f(x, y)
    assert e.value.code == 6 and "tensor<8xf32>" in str(e.value)
    with pytest.raises(rx.ReactantError):
        f(x)
    z = rx.to_rarray(np.zeros(16, np.float64), client)
    with pytest.raises(rx.ReactantError) as e:
        f(x, z)
    assert e.value.code == 6


def test_buffer_round_trip_and_allocator_stats(rx, client):
    dev = client.addressable_devices[0]
    for dt in (np.float32, np.int32, np.bool_, np.float64, np.int64, np.uint8):
        a = (np.arange(2 * 3 * 5).reshape(2, 3, 5) % 7).astype(dt)
        r = rx.to_rarray(a, client)
        assert r.data[0].dims == (5, 3, 2), "dims cross the boundary reversed"
        assert np.array_equal(np.asarray(r), a)
    s = dev.allocator_stats()
    assert s["bytes_in_use"] >= 0 and s["peak_bytes_in_use"] > 0 and s["bytes_limit"] > 0
    assert client.platform_name == "cuda"


def test_compiling_a_module_again_reuses_its_plan(rx, client):
    from reactant_jl_b200 import _lib
    text = rx.programs.sinsum_add(12345)
    before = _lib.lib().RxPlanCacheHits()
    f = rx.compile(text, client)
    g = rx.compile(text, client)
    assert _lib.lib().RxPlanCacheHits() >= before + 1
    x = np.linspace(-1, 1, 12345, dtype=np.float32)
    a, b = float(f(rx.to_rarray(x, client), rx.to_rarray(x, client))), float(g(rx.to_rarray(x, client), rx.to_rarray(x, client)))
    assert a == b


# ---------------------------------------------------------------- scans (cumsum and friends)
@pytest.mark.parametrize("dims,axis", [((1,), 0), ((33,), 0), ((5000,), 0), (((1 << 20) + 3,), 0), ((700, 5000), 1), ((3, 300000), 1),
                                        ((257, 129), 0), ((6, 1000, 7), 1), ((4, 5, 2049), 2), ((70000, 3), 1)])
@pytest.mark.parametrize("kind", ["add", "maximum"])
def test_scans_along_one_dimension(rx, ref, client, dims, axis, kind):
    rng = np.random.default_rng(len(dims) * 100 + axis)
    x = rng.standard_normal(dims).astype(np.float32)
    text = rx.programs.scan(dims, axis, kind)
    (got,), _, _ = run(rx, client, text, [x])
    want = ref.run_module(text, [x])[0]
    if kind == "maximum":
        assert np.array_equal(got, want)
    else:
        n = dims[axis]
        # a prefix of k terms carries the reduction bound for k terms, relative to the 2-norm of the terms seen so far
        norm = np.sqrt(np.cumsum(x.astype(np.float64) ** 2, axis=axis))
        assert np.all(np.abs(got - want) <= ref.reduction_tolerance(max(n, 2)) * np.maximum(np.abs(want), norm) + 1e-30)


def test_integer_scans_are_exact(rx, ref, client):
    x = np.random.default_rng(0).integers(-1000, 1000, size=(37, 4099)).astype(np.int32)
    for axis in (0, 1):
        for kind in ("add", "minimum"):
            text = rx.programs.scan(x.shape, axis, kind, et="i32")
            (got,), _, _ = run(rx, client, text, [x])
            assert np.array_equal(got, ref.run_module(text, [x])[0])


def test_an_exported_bundle_runs_from_its_files(rx, ref, client, tmp_path):
    """The file layout of Reactant.Serialization.export_to_enzymejax: <name>_0.mlir + <name>_0_inputs.npz with
    arr_1..arr_n in the row-major layout of the module's argument types."""
    rows, cols = 96, 40
    text = rx.programs.logsumexp_dims1(rows, cols)
    x = np.random.default_rng(5).standard_normal((cols, rows)).astype(np.float32)   # boundary layout of the argument
    (tmp_path / "lse_0.mlir").write_text(text)
    np.savez_compressed(tmp_path / "lse_0_inputs.npz", arr_1=x)
    thunk, inputs = rx.load_export(str(tmp_path), "lse", client=client)
    got = np.asarray(thunk(*inputs)).T
    want = ref.run_module(text, [x])[0]
    np.testing.assert_allclose(got, want, rtol=ref.reduction_tolerance(rows))


def test_more_elementwise_ops(rx, ref, client):
    """tan, cbrt, both roundings, is_finite, atan2, remainder (src/Ops.jl:398-460, 536-589)."""
    n = 4099
    t, ti = f"tensor<{n}xf32>", f"tensor<{n}xi1>"
    text = module([t, t], [t, t, ti], f"""    %0 = stablehlo.tan %arg0 : {t}
    %1 = stablehlo.cbrt %arg1 : {t}
    %2 = stablehlo.add %0, %1 : {t}
    %3 = stablehlo.round_nearest_even %arg1 : {t}
    %4 = stablehlo.round_nearest_afz %arg1 : {t}
    %5 = stablehlo.subtract %3, %4 : {t}
    %6 = stablehlo.atan2 %arg0, %arg1 : {t}
    %7 = stablehlo.remainder %arg1, %arg0 : {t}
    %8 = stablehlo.add %6, %7 : {t}
    %9 = stablehlo.add %8, %5 : {t}
    %10 = stablehlo.divide %arg0, %5 : {t}
    %11 = stablehlo.is_finite %10 : ({t}) -> {ti}
    return %2, %9, %11 : {t}, {t}, {ti}""")
    rng = np.random.default_rng(3)
    x = rng.uniform(-1.4, 1.4, n).astype(np.float32)
    y = (rng.integers(-40, 40, n) * 0.25).astype(np.float32)   # quarters: exercises both tie rules exactly
    got, _, _ = run(rx, client, text, [x, y])
    want = ref.run_module(text, [x, y])
    np.testing.assert_allclose(got[0], want[0], rtol=4e-6, atol=1e-6)
    np.testing.assert_allclose(got[1], want[1], rtol=4e-6, atol=2e-6)
    assert np.array_equal(got[2], want[2])


def test_thunks_called_from_several_host_threads(rx, ref, client):
    """Julia tasks may call compiled functions from any OS thread (different Thunks concurrently, and finalizers at any
    time): executions on one device are serialised inside the library and every call returns its own result."""
    import threading
    n = 1 << 16
    rng = np.random.default_rng(11)
    x = rng.uniform(-3, 3, n).astype(np.float32)
    y = rng.uniform(-3, 3, n).astype(np.float32)
    f_sum = rx.compile(rx.programs.sinsum_add(n), client)
    rows, cols = 512, 96
    a = rng.standard_normal((rows, cols)).astype(np.float32)
    f_lse = rx.compile(rx.programs.logsumexp_dims1(rows, cols), client)
    want_sum = float(f_sum(rx.to_rarray(x, client), rx.to_rarray(y, client)))
    want_lse = np.asarray(f_lse(rx.to_rarray(a, client)))
    errors = []

    def worker(kind):
        try:
            for _ in range(40):
                if kind == 0:
                    got = float(f_sum(rx.to_rarray(x, client), rx.to_rarray(y, client)))
                    assert got == want_sum, (got, want_sum)       # deterministic reduction: same bits every time
                else:
                    got = np.asarray(f_lse(rx.to_rarray(a, client)))
                    assert np.array_equal(got, want_lse)
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(k % 2,)) for k in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
