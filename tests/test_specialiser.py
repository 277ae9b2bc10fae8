"""Run-time specialisation of fused chains: the generated kernels must compile for sm_100a (checked without a
device, NVRTC only) and must produce the same bits as the on-GPU interpreter they replace."""
import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()
P = rx.programs


CHAIN_MODULE = """
module {
  func.func @main(%x: tensor<1024x2048xf32>, %y: tensor<1024x2048xf32>, %s: tensor<2048xf32>) -> (tensor<1024x2048xf32>, tensor<2048xf32>, tensor<f32>) {
    %c = stablehlo.constant dense<5.000000e-01> : tensor<1024x2048xf32>
    %z = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %sb = stablehlo.broadcast_in_dim %s, dims = [1] : (tensor<2048xf32>) -> tensor<1024x2048xf32>
    %0 = stablehlo.tanh %x : tensor<1024x2048xf32>
    %1 = stablehlo.multiply %0, %sb : tensor<1024x2048xf32>
    %2 = stablehlo.subtract %y, %1 : tensor<1024x2048xf32>
    %3 = stablehlo.multiply %2, %2 : tensor<1024x2048xf32>
    %4 = stablehlo.compare GT, %3, %c : (tensor<1024x2048xf32>, tensor<1024x2048xf32>) -> tensor<1024x2048xi1>
    %5 = stablehlo.select %4, %3, %1 : tensor<1024x2048xi1>, tensor<1024x2048xf32>
    %6 = stablehlo.divide %c, %5 : tensor<1024x2048xf32>
    %7 = stablehlo.maximum %6, %2 : tensor<1024x2048xf32>
    %col = stablehlo.reduce(%7 init: %z) applies stablehlo.add across dimensions = [0] : (tensor<1024x2048xf32>, tensor<f32>) -> tensor<2048xf32>
    %all = stablehlo.reduce(%3 init: %z) applies stablehlo.add across dimensions = [0, 1] : (tensor<1024x2048xf32>, tensor<f32>) -> tensor<f32>
    return %7, %col, %all : tensor<1024x2048xf32>, tensor<2048xf32>, tensor<f32>
  }
}
"""


# minimum of a minimum and a product of the same operand: as nested selects around fminf this shape crashed the
# run-time compiler, which took the calling process with it
NESTED_MIN_MODULE = """
module {
  func.func @main(%v: tensor<64xf32>) -> tensor<64x130x3xf32> {
    %bc = stablehlo.broadcast_in_dim %v, dims = [0] : (tensor<64xf32>) -> tensor<64x130x3xf32>
    %k = stablehlo.constant dense<1.5845897197723389> : tensor<64x130x3xf32>
    %0 = stablehlo.multiply %bc, %k : tensor<64x130x3xf32>
    %1 = stablehlo.minimum %k, %bc : tensor<64x130x3xf32>
    %2 = stablehlo.minimum %0, %1 : tensor<64x130x3xf32>
    %3 = stablehlo.abs %2 : tensor<64x130x3xf32>
    return %3 : tensor<64x130x3xf32>
  }
}
"""


def _programs():
    return {
        "nested_min": NESTED_MIN_MODULE,
        "sinsum_add": P.sinsum_add(1 << 12),
        "logsumexp_raw": P.logsumexp_dims1(64, 256, raw=True),
        "jacobi_dus": P.jacobi2d(64, 3),
        "mlp_grad": P.mlp_grad(128, 256, 128, 128),
        "chain": CHAIN_MODULE,
    }


@pytest.mark.parametrize("name", list(_programs()))
def test_every_chain_compiles_for_sm100a(name):
    built = rx.specialise_check(_programs()[name])
    if name not in ("jacobi_dus", "logsumexp_raw"):  # these plan into the dedicated stencil / logsumexp kernels
        assert built, "no chain kernels were generated"
    for k in built:
        assert k["cubin_bytes"] > 0, k


def test_generated_code_is_built_from_the_interpreter_tables():
    # comparison directions, immediates and the reversed forms all reach the generated source
    built = rx.specialise_check(CHAIN_MODULE)
    families = {k["kernel"] for k in built}
    assert "k_map_rows<rx::SpecChain, 2>" in families
    assert "k_reduce_col_vec<rx::SpecChain>" in families
    assert "k_reduce_full_rows<rx::SpecChain>" in families


@pytest.mark.gpu
def test_specialised_kernels_match_the_interpreter_bit_for_bit():
    rng = np.random.default_rng(7)
    x = rng.standard_normal((1024, 2048), dtype=np.float32)
    y = rng.standard_normal((1024, 2048), dtype=np.float32)
    s = rng.standard_normal((2048,), dtype=np.float32)
    oracle, _ = entry.load_oracle()
    want = oracle.run_module(CHAIN_MODULE, [x, y, s])
    outs = {}
    try:
        for mode, threshold in (("interpreter", -1), ("specialised", 0)):
            rx.chain_specialiser(threshold)
            before = rx.chain_specialiser_stats()
            f = rx.compile(CHAIN_MODULE)
            # host arrays follow the reversed-dimension (column-major) convention of the boundary
            r = f(rx.to_rarray(x.T), rx.to_rarray(y.T), rx.to_rarray(s))
            outs[mode] = [np.ascontiguousarray(np.asarray(t).T) for t in r]
            after = rx.chain_specialiser_stats()
            if mode == "specialised":
                assert not after["unavailable"], "NVRTC or the driver entry points could not be loaded on a GPU machine"
                assert after["compiled"] + after["cache_hits"] > before["compiled"] + before["cache_hits"]
                assert after["failed"] == 0
            else:
                assert after["compiled"] == before["compiled"] and after["cache_hits"] == before["cache_hits"]
    finally:
        rx.chain_specialiser(1 << 20)
    for a, b in zip(outs["interpreter"], outs["specialised"]):
        assert a.dtype == b.dtype and a.shape == b.shape
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # and both agree with the oracle.  The select is discontinuous where %3 crosses 0.5: elements within a few ulp
    # of the threshold may legitimately take the other branch (tanh differs in the last bit between libraries).
    t = np.tanh(x.astype(np.float64)) * s.astype(np.float64)
    margin = np.abs((y - t) ** 2 - 0.5)
    safe = margin > 1e-5
    assert safe.mean() > 0.9999
    np.testing.assert_allclose(outs["specialised"][0][safe], want[0][safe], rtol=2e-6, atol=1e-6)
    cols_ok = safe.all(axis=0)
    tol = oracle.reduction_tolerance(1024)
    np.testing.assert_allclose(outs["specialised"][1][cols_ok], want[1][cols_ok], rtol=tol, atol=tol * np.abs(want[0]).sum(axis=0).max())
    tol = oracle.reduction_tolerance(1024 * 2048)
    np.testing.assert_allclose(outs["specialised"][2], want[2], rtol=tol)


# Two chains where a constant written as a literal let the run-time compiler change the result: it evaluated
# tanh(c) itself (one ulp away from the device's tanhf), and it strength-reduced x * -256 under a signed minimum to
# the minimum of x * 256.  Constants are therefore read from the program at run time.
CONST_TANH_MODULE = """
module {
  func.func @main(%x: tensor<130x1024xf32>) -> tensor<130x1024xf32> {
    %k = stablehlo.constant dense<0.7570777535438538> : tensor<130x1024xf32>
    %t = stablehlo.tanh %k : tensor<130x1024xf32>
    %0 = stablehlo.add %x, %t : tensor<130x1024xf32>
    %1 = stablehlo.minimum %t, %0 : tensor<130x1024xf32>
    return %1 : tensor<130x1024xf32>
  }
}
"""
CONST_IMUL_MIN_MODULE = """
module {
  func.func @main(%x: tensor<128x16x16xi32>) -> tensor<i32> {
    %k = stablehlo.constant dense<-256> : tensor<128x16x16xi32>
    %m = stablehlo.multiply %x, %k : tensor<128x16x16xi32>
    %z = stablehlo.constant dense<2147483647> : tensor<i32>
    %r = stablehlo.reduce(%m init: %z) applies stablehlo.minimum across dimensions = [0, 1, 2] : (tensor<128x16x16xi32>, tensor<i32>) -> tensor<i32>
    return %r : tensor<i32>
  }
}
"""
# min(acc, min(-x, t)) in a reduction loop and -max(a, max(a, b)): a signed integer min / max next to a negation
# lost the negation of one operand; signed min / max are computed on sign-biased unsigned values since.
NEG_UNDER_MIN_MODULE = """
module {
  func.func @main(%x: tensor<5x2048xi32>) -> tensor<2048xi32> {
    %io = stablehlo.iota dim = 1 : tensor<5x2048xi32>
    %a = stablehlo.abs %io : tensor<5x2048xi32>
    %n = stablehlo.negate %x : tensor<5x2048xi32>
    %m = stablehlo.minimum %a, %n : tensor<5x2048xi32>
    %z = stablehlo.constant dense<2147483647> : tensor<i32>
    %r = stablehlo.reduce(%m init: %z) applies stablehlo.minimum across dimensions = [0] : (tensor<5x2048xi32>, tensor<i32>) -> tensor<2048xi32>
    return %r : tensor<2048xi32>
  }
}
"""
NEGATED_MAX_MODULE = """
module {
  func.func @main(%x: tensor<2x16x1xi32>) -> tensor<2x16x1xi32> {
    %k = stablehlo.constant dense<3> : tensor<2x16x1xi32>
    %v0 = stablehlo.negate %k : tensor<2x16x1xi32>
    %z0 = stablehlo.subtract %v0, %v0 : tensor<2x16x1xi32>
    %p = stablehlo.compare NE, %z0, %x : (tensor<2x16x1xi32>, tensor<2x16x1xi32>) -> tensor<2x16x1xi1>
    %v2 = stablehlo.select %p, %v0, %k : tensor<2x16x1xi1>, tensor<2x16x1xi32>
    %v3 = stablehlo.maximum %v2, %v0 : tensor<2x16x1xi32>
    %v6 = stablehlo.maximum %v2, %v3 : tensor<2x16x1xi32>
    %v9 = stablehlo.negate %v6 : tensor<2x16x1xi32>
    return %v9 : tensor<2x16x1xi32>
  }
}
"""


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tanh_of_constant", "multiply_by_constant_under_min", "negation_under_min", "negated_max"])
def test_constants_and_negations_do_not_let_the_compiler_change_results(name):
    rng = np.random.default_rng(11)
    if name == "tanh_of_constant":
        text, x = CONST_TANH_MODULE, rng.uniform(-1.5, 1.5, size=(130, 1024)).astype(np.float32)
    elif name == "negation_under_min":
        text, x = NEG_UNDER_MIN_MODULE, rng.integers(-60, 60, size=(5, 2048)).astype(np.int32)
    elif name == "negated_max":
        text, x = NEGATED_MAX_MODULE, rng.integers(-2, 3, size=(2, 16, 1)).astype(np.int32)
    else:
        text = CONST_IMUL_MIN_MODULE
        x = rng.integers(-60, 60, size=(128, 16, 16)).astype(np.int32)
        x.ravel()[rng.integers(0, x.size, size=400)] = rng.choice(np.array([65535, -65536, 2**31 - 1, -(2**31), 2**30], dtype=np.int64), size=400).astype(np.int32)
    outs = []
    try:
        for threshold in (-1, 0):
            rx.chain_specialiser(threshold)
            r = rx.compile(text)(rx.to_rarray(np.ascontiguousarray(x.T)))
            outs.append(np.ascontiguousarray(np.asarray(r).T))
    finally:
        rx.chain_specialiser(1 << 20)
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    if name == "multiply_by_constant_under_min":
        want = (x.astype(np.int64) * -256 & 0xFFFFFFFF).astype(np.uint32).view(np.int32).min()
        assert int(outs[1]) == int(want)
    if name == "negated_max":
        assert np.array_equal(outs[1], np.where(x != 0, 3, -3).astype(np.int32))
    if name == "negation_under_min":
        want = np.minimum(np.arange(2048, dtype=np.int32)[None, :], -x).min(axis=0)
        assert np.array_equal(outs[1], want)


@pytest.mark.gpu
def test_default_threshold_keeps_small_launches_on_the_interpreter():
    rx.chain_specialiser(1 << 20)
    before = rx.chain_specialiser_stats()
    n = 1 << 12
    x = np.linspace(0, 1, n, dtype=np.float32)
    f = rx.compile("""
module {
  func.func @main(%x: tensor<4096xf32>) -> tensor<4096xf32> {
    %0 = stablehlo.cosine %x : tensor<4096xf32>
    %1 = stablehlo.multiply %0, %x : tensor<4096xf32>
    return %1 : tensor<4096xf32>
  }
}
""")
    got = np.asarray(f(rx.to_rarray(x)))
    after = rx.chain_specialiser_stats()
    assert after["compiled"] == before["compiled"] and after["cache_hits"] == before["cache_hits"]
    np.testing.assert_allclose(got, np.cos(x) * x, rtol=2e-6, atol=1e-7)


@pytest.mark.gpu
def test_compiled_chains_persist_across_processes(tmp_path):
    """With RX_JIT_CACHE_DIR set, a second process loads the cubin of a chain instead of compiling it, and computes
    the same bits."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "chain_once.py"
    script.write_text(f"""
import sys, json, numpy as np
sys.path.insert(0, {root!r})
import __graft_entry__ as entry
rx = entry.load_package()
rx.chain_specialiser(0)
t = "tensor<4096xf32>"
text = ("module {{\\n  func.func @main(%x: " + t + ") -> " + t + " {{\\n    %0 = stablehlo.tanh %x : " + t +
        "\\n    %1 = stablehlo.multiply %0, %x : " + t + "\\n    return %1 : " + t + "\\n  }}\\n}}\\n")
x = np.linspace(-2, 2, 4096, dtype=np.float32)
y = np.asarray(rx.compile(text)(rx.to_rarray(x)))
print(json.dumps({{"stats": rx.chain_specialiser_stats(), "bits": int(y.view(np.uint32).astype(np.uint64).sum())}}))
""")
    cache = tmp_path / "cache"
    cache.mkdir()
    env = dict(os.environ, RX_JIT_CACHE_DIR=str(cache))
    outs = []
    for _ in range(2):
        r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(json.loads(r.stdout.strip().splitlines()[-1]))
    first, second = outs
    assert first["stats"]["compiled"] >= 1 and first["stats"]["disk_hits"] == 0
    assert second["stats"]["compiled"] == 0 and second["stats"]["disk_hits"] >= 1
    assert first["bits"] == second["bits"]
    assert any(f.startswith("rx_chain_") for f in os.listdir(cache))
