"""Elementwise and reduction work fused into the epilogue of the tensor-core GEMM that produces its operand.

CPU: the planner's decisions (what joins a GEMM, what does not, which products are no longer stored) and that the
kernel compiles around each chain without a device.  GPU: with the fusion on and off (RX_GEMM_EPILOGUE=0) the
elementwise results are the same bits, the sums agree within the fp32 reduction tolerance, and both agree with
the oracle."""
import numpy as np
import pytest


def kinds(plan):
    return [s["kind"] for s in plan["steps"]]


def bias_gelu_module(M, N, K, with_sum=False):
    """z = bf16(A * B) + b; h = gelu_tanh(z); results: bf16(h) and, optionally, the column sums of h."""
    ta, tb, tz, tzf, tbias = f"tensor<{M}x{K}xbf16>", f"tensor<{K}x{N}xbf16>", f"tensor<{M}x{N}xbf16>", f"tensor<{M}x{N}xf32>", f"tensor<{N}xf32>"
    res = f"{tz}, {tbias}" if with_sum else tz
    body = f"""    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : ({ta}, {tb}) -> {tz}
    %1 = stablehlo.convert %0 : ({tz}) -> {tzf}
    %2 = stablehlo.broadcast_in_dim %arg2, dims = [1] : ({tbias}) -> {tzf}
    %3 = stablehlo.add %1, %2 : {tzf}
    %4 = "enzymexla.math.gelu"(%3) <{{gelu_approximation = #enzymexla<gelu_approximation TANH>}}> : ({tzf}) -> {tzf}
    %5 = stablehlo.convert %4 : ({tzf}) -> {tz}
"""
    if with_sum:
        body += f"    %6 = stablehlo.reduce(%4 init: %cst) applies stablehlo.add across dimensions = [0] : ({tzf}, tensor<f32>) -> {tbias}\n    return %5, %6 : {res}"
    else:
        body += f"    return %5 : {res}"
    return f"module {{\n  func.func @main(%arg0: {ta}, %arg1: {tb}, %arg2: {tbias}) -> ({res}) {{\n{body}\n  }}\n}}\n"


def test_mlp_step_plans_as_five_gemms_with_fused_epilogues(rx, monkeypatch):
    monkeypatch.delenv("RX_GEMM_EPILOGUE", raising=False)
    p = rx.plan_describe(rx.programs.mlp_grad())
    assert kinds(p) == ["gemm", "gemm", "sum_partials", "gemm", "gemm", "sum_partials", "gemm", "map"], p
    epi = [s.get("epilogue") for s in p["steps"] if s["kind"] == "gemm"]
    assert epi[0] == {"instrs": 13, "leaves": 2, "results": 2, "column_sums": 0, "full_sums": 0}   # product (read again by the backward pass) + gelu as bf16
    assert epi[1]["results"] == 1 and epi[1]["column_sums"] == 1 and epi[1]["full_sums"] == 1       # bf16 MSE gradient, bias gradient, loss; the product is not stored
    assert epi[2] is None and epi[4] is None                                                        # weight gradients: plain products
    assert epi[3]["results"] == 1 and epi[3]["column_sums"] == 1                                    # gelu' gradient as bf16 + bias gradient
    monkeypatch.setenv("RX_GEMM_EPILOGUE", "0")
    q = rx.plan_describe(rx.programs.mlp_grad())
    assert kinds(q).count("gemm") == 5 and "sum_partials" not in kinds(q) and kinds(q).count("map") == 4


def test_what_does_not_join_a_gemm(rx, monkeypatch):
    monkeypatch.delenv("RX_GEMM_EPILOGUE", raising=False)
    # small products run on other kernels: nothing is fused
    assert kinds(rx.plan_describe(bias_gelu_module(128, 128, 64))) == ["gemm", "map"]
    # a transposed read of the product cannot be evaluated at (m, n)
    M = 256
    t, tf = f"tensor<{M}x{M}xbf16>", f"tensor<{M}x{M}xf32>"
    text = f"""module {{
  func.func @main(%arg0: {t}, %arg1: {t}) -> {tf} {{
    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : ({t}, {t}) -> {t}
    %1 = stablehlo.convert %0 : ({t}) -> {tf}
    %2 = stablehlo.transpose %1, dims = [1, 0] : ({tf}) -> {tf}
    %3 = stablehlo.add %1, %2 : {tf}
    return %3 : {tf}
  }}
}}
"""
    assert kinds(rx.plan_describe(text)) == ["gemm", "map"]
    # a maximum over the columns is not an additive reduction: the chain joins, the reduction stays a kernel of its own
    text = bias_gelu_module(256, 256, 64, with_sum=True).replace("applies stablehlo.add", "applies stablehlo.maximum").replace("dense<0.000000e+00>", "dense<0xFF800000>")
    k = kinds(rx.plan_describe(text))
    assert k[0] == "gemm" and "sum_partials" not in k and any(x.startswith("reduce") for x in k)


def test_fused_kernels_compile_without_a_device(rx, monkeypatch):
    monkeypatch.delenv("RX_GEMM_EPILOGUE", raising=False)
    out = rx.specialise_check(bias_gelu_module(512, 256, 128, with_sum=True))
    names = [o["kernel"] for o in out]
    assert any(n.startswith("k_gemm_pair<true") for n in names) and any(n.startswith("k_gemm_pair<false") for n in names)
    assert all(o["cubin_bytes"] > 0 for o in out)


def _run(rx, client, text, ins_bf16, bias):
    f = rx.compile(text, client)
    args = [rx.to_rarray(a.T.astype(rx.bfloat16), client) for a in ins_bf16] + [rx.to_rarray(bias, client)]
    out = f(*args)
    outs = out if isinstance(out, tuple) else (out,)
    return [np.asarray(o).T.astype(np.float32) for o in outs], f


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 200), (1024, 4096, 1024), (4096, 1024, 512), (288, 320, 72)])
def test_bias_gelu_epilogue_matches_the_separate_kernels_bit_for_bit(rx, ref, client, monkeypatch, M, N, K):
    rng = np.random.default_rng(M + N + K)
    A = ref.round_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    B = ref.round_to_bf16((rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32))
    bias = rng.standard_normal(N).astype(np.float32)
    text = bias_gelu_module(M, N, K, with_sum=True)
    monkeypatch.setenv("RX_GEMM_EPILOGUE", "0")
    (h0, s0), f0 = _run(rx, client, text, [A, B], bias)
    assert all("epilogue" not in s for s in f0.describe()["steps"])
    monkeypatch.delenv("RX_GEMM_EPILOGUE")
    (h1, s1), f1 = _run(rx, client, text, [A, B], bias)
    steps = f1.describe()["steps"]
    assert [s["kind"] for s in steps] == ["gemm", "sum_partials"] and steps[0]["epilogue"]["column_sums"] == 1
    assert np.array_equal(h0, h1), "same chain, same roundings: the fused epilogue must give the same bits"
    want_h, want_s = ref.run_module(text, [A, B, bias])
    assert np.abs(h1 - want_h).max() <= 2e-2 * np.abs(want_h).max()
    tol = ref.reduction_tolerance(M) * np.sqrt((want_h.astype(np.float64) ** 2).sum(axis=0)).max() + 2e-2 * np.abs(want_s).max()
    assert np.abs(s1 - want_s).max() <= tol and np.abs(s0 - s1).max() <= 1e-4 * np.abs(want_s).max() + 1e-5
    # deterministic: the ordered second pass gives the same bits on every run
    (h2, s2), _ = _run(rx, client, text, [A, B], bias)
    assert np.array_equal(s1, s2) and np.array_equal(h1, h2)


@pytest.mark.gpu
@pytest.mark.parametrize("F,H,O,B", [(256, 512, 256, 512), (320, 768, 288, 384), (1024, 4096, 1024, 4096)])
def test_mlp_step_fused_against_unfused_and_oracle(rx, ref, client, monkeypatch, F, H, O, B):
    rng = np.random.default_rng(6)
    bf = lambda a: ref.round_to_bf16(a.astype(np.float32))
    W1, W2 = bf(rng.standard_normal((F, H)) / np.sqrt(F)), bf(rng.standard_normal((H, O)) / np.sqrt(H))
    b1, b2 = (0.01 * rng.standard_normal(H)).astype(np.float32), (0.01 * rng.standard_normal(O)).astype(np.float32)
    X, Y = bf(rng.standard_normal((B, F))), rng.standard_normal((B, O)).astype(np.float32)
    text = rx.programs.mlp_grad(F, H, O, B)
    up = lambda a, bf16: rx.to_rarray(a.T.astype(rx.bfloat16) if bf16 else a.T, client)

    def run():
        f = rx.compile(text, client)
        outs = f(up(W1, True), up(b1, False), up(W2, True), up(b2, False), up(X, True), up(Y, False))
        return [np.asarray(o).T.astype(np.float32) for o in outs], f

    monkeypatch.setenv("RX_GEMM_EPILOGUE", "0")
    plain, f0 = run()
    monkeypatch.delenv("RX_GEMM_EPILOGUE")
    fused, f1 = run()
    k0, k1 = [s["kind"] for s in f0.describe()["steps"]], [s["kind"] for s in f1.describe()["steps"]]
    assert "sum_partials" not in k0 and k1.count("sum_partials") == 2 and k1.count("map") == 1 and len(k1) == 8
    names = ("dW1", "db1", "dW2", "db2", "loss")
    # the weight gradients are products of operands that the two forms compute with identical roundings
    assert np.array_equal(plain[0], fused[0]) and np.array_equal(plain[2], fused[2])
    want = ref.run_module(text, [W1, b1, W2, b2, X, Y]) if B <= 1024 else None
    for name, p_, f_, k in zip(names, plain, fused, range(5)):
        scale = np.abs(p_).max()
        assert np.abs(p_ - f_).max() <= 1e-4 * scale, (name, np.abs(p_ - f_).max(), scale)   # sums: same terms, different fixed orders
        if want is not None:
            assert np.abs(f_ - want[k]).max() <= 2e-2 * np.abs(want[k]).max(), name
