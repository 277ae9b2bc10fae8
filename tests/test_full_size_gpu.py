"""Parity at the full sizes of the benchmark configurations that the smaller parity tests do not reach:
the sharded-sinsum vector of 2^30 pairs (on one GPU), the MLP step at 1024 x 4096 x 1024 x 4096, and the
two-half-step spelling of the Jacobi loop at 8192^2.  Tolerances are the benchmark contract's: 1e-5*sqrt(log2 n)
for fp32 reductions (relative to the 2-norm of the terms, the sum being ill-conditioned), 2e-2 of the largest
magnitude for anything behind a bf16 dot_general, bit-exact for the stencil."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_sinsum_2p30_against_the_chunked_float64_sum(rx, ref, cpu, client):
    n, chunks = 1 << 30, 8
    step = n // chunks
    x = np.empty(n, np.float32)
    y = np.empty(n, np.float32)
    total, sumsq = 0.0, 0.0
    cpu.set_threads()
    for c in range(chunks):  # eight independently seeded chunks, the float64 ground truth summed chunk by chunk
        rng = np.random.default_rng(1100 + c)
        sl = slice(c * step, (c + 1) * step)
        x[sl] = rng.random(step, dtype=np.float32) * np.float32(2 * np.pi) - np.float32(np.pi)
        y[sl] = rng.random(step, dtype=np.float32) * np.float32(2 * np.pi) - np.float32(np.pi)
        s, q = cpu.sinsum_add_f64(x[sl], y[sl])
        total += s
        sumsq += q
    f = rx.compile(rx.programs.sinsum_add(n), client)
    X, Y = rx.to_rarray(x, client), rx.to_rarray(y, client)
    got = float(f(X, Y))
    tol = 1e-5 * math.sqrt(30)
    assert tol == pytest.approx(ref.reduction_tolerance(n))
    assert abs(got - total) <= tol * max(abs(total), math.sqrt(sumsq)), (got, total)
    assert float(f(X, Y)) == got, "the ordered cross-CTA combine gives the same bits on every run"
    # linearity: the sum over the two halves, each reduced on its own, differs from the whole by rounding only
    h = n // 2
    g = rx.compile(rx.programs.sinsum_add(h), client)
    parts = float(g(rx.to_rarray(x[:h], client), rx.to_rarray(y[:h], client))) + float(g(rx.to_rarray(x[h:], client), rx.to_rarray(y[h:], client)))
    assert abs(parts - got) <= tol * math.sqrt(sumsq)


def test_mlp_step_at_the_benchmark_shape(rx, ref, client):
    F, H, O, B = 1024, 4096, 1024, 4096
    rng = np.random.default_rng(6)
    bf = lambda a: ref.round_to_bf16(a.astype(np.float32))
    W1 = bf(rng.standard_normal((F, H)) / np.sqrt(F))
    W2 = bf(rng.standard_normal((H, O)) / np.sqrt(H))
    b1 = (0.01 * rng.standard_normal(H)).astype(np.float32)
    b2 = (0.01 * rng.standard_normal(O)).astype(np.float32)
    X = bf(rng.standard_normal((B, F)))
    Y = rng.standard_normal((B, O)).astype(np.float32)
    ins = [W1, b1, W2, b2, X, Y]
    text = rx.programs.mlp_grad(F, H, O, B)
    f = rx.compile(text, client)
    assert [s["kind"] for s in f.describe()["steps"]].count("gemm") == 5
    up = lambda a, bf16: rx.to_rarray(a.T.astype(rx.bfloat16) if bf16 else a.T, client)
    outs = f(up(W1, True), up(b1, False), up(W2, True), up(b2, False), up(X, True), up(Y, False))
    got = [np.asarray(o).T.astype(np.float32) for o in outs]
    want = ref.run_module(text, ins)  # float64 accumulation, bf16 roundings where the module has them
    for name, g, w in zip(("dW1", "db1", "dW2", "db2", "loss"), got, want):
        scale = float(np.abs(w).max())
        assert g.shape == w.shape
        assert float(np.abs(g - w).max()) <= 2e-2 * scale, (name, float(np.abs(g - w).max()), scale)
    # the loss is a plain fp32 reduction of 2^22 squared differences behind one bf16 GEMM: far inside 2e-2
    assert abs(float(got[4]) - float(want[4])) <= 2e-3 * abs(float(want[4]))


@pytest.mark.parametrize("n,iters", [(1028, 3), (8192, 2)])
def test_jacobi_two_half_steps_per_iteration_bit_exact(rx, ref, cpu, client, n, iters):
    """The spelling of the reference's own benchmark: B from A, then A from B, in every iteration.  Both updates run
    in place (no copy of either array) and the whole loop is one cooperative launch."""
    rng = np.random.default_rng(n)
    a = rng.random((n, n), dtype=np.float32)
    b = rng.random((n, n), dtype=np.float32)
    text = rx.programs.jacobi2d(n, iters, form="halfsteps")
    f = rx.compile(text, client)
    plan = f.describe()
    assert plan["slots"] == 2 and [s["kind"] for s in plan["steps"][0]["body"]] == ["stencil", "stencil"], plan
    dev = client.addressable_devices[0]
    A, B = rx.to_rarray(a.T, client), rx.to_rarray(b.T, client)
    before = dev.kernel_launches()
    ra, rb = f(A, B)
    assert dev.kernel_launches() - before == 1
    ga, gb = np.asarray(ra).T, np.asarray(rb).T
    wa, wb = cpu.jacobi2d(a, b, 2 * iters, "polybench")
    assert np.array_equal(ga, wa) and np.array_equal(gb, wb)
    if n <= 2048:  # the numpy interpreter of the module text agrees with the C restatement
        na, nb = ref.run_module(text, [a, b])
        assert np.array_equal(na, wa) and np.array_equal(nb, wb)


def test_float_to_int_conversion_saturates(rx, ref, client):
    t, ti = "tensor<8xf32>", "tensor<8xi32>"
    text = f"module {{\n  func.func @main(%arg0: {t}) -> ({ti}) {{\n    %0 = stablehlo.convert %arg0 : ({t}) -> {ti}\n    return %0 : {ti}\n  }}\n}}\n"
    x = np.array([2147483648.0, 3e9, np.inf, -2147483648.0, -3e9, -np.inf, np.nan, 2147483520.0], np.float32)
    f = rx.compile(text, client)
    got = np.asarray(f(rx.to_rarray(x, client)))
    want = np.array([2147483647, 2147483647, 2147483647, -2147483648, -2147483648, -2147483648, 0, 2147483520], np.int32)
    assert np.array_equal(got, want), got
    with np.errstate(all="ignore"):
        assert np.array_equal(ref.run_module(text, [x])[0], want)
