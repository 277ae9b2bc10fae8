"""bf16 dot_general over randomly drawn shapes and all four operand layouts (the forward product and the three
transposed contractions of its gradient), against the float64 product of the same bf16 inputs.  Shapes include
extents that are not multiples of the tile, of the 64-element copy group or of the 16-byte pitch rule, so the
two-CTA wide-slab kernel, its narrow form, the one-CTA kernel and the CUDA-core path all get exercised; f32
output (accumulator written unrounded) is covered as well."""
import numpy as np
import pytest

import __graft_entry__ as entry

rx = entry.load_package()


def dot_module(lhs_shape, rhs_shape, lc, rc, out_shape, et, out_et):
    """out_et == "f32" with bf16 operands: the contraction's own result type is f32 (accumulator written unrounded)."""
    tl = f"tensor<{lhs_shape[0]}x{lhs_shape[1]}x{et}>"
    tr = f"tensor<{rhs_shape[0]}x{rhs_shape[1]}x{et}>"
    to = f"tensor<{out_shape[0]}x{out_shape[1]}x{out_et}>"
    body = f"    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [{lc}] x [{rc}], precision = [DEFAULT, DEFAULT] : ({tl}, {tr}) -> {to}\n"
    body += f"    return %0 : {to}\n"
    return f"module {{\n  func.func @main(%arg0: {tl}, %arg1: {tr}) -> {to} {{\n{body}  }}\n}}\n"


def cases():
    rng = np.random.default_rng(2024)
    out = []
    nice = [64, 128, 256, 320, 512, 768]
    for i in range(40):
        if i % 3 == 0:
            m, n, k = (int(rng.choice(nice)) for _ in range(3))
        elif i % 3 == 1:
            m, n, k = (int(rng.integers(1, 90)) * 8 for _ in range(3))  # pitch rule holds, tiles ragged
        else:
            m, n, k = (int(rng.integers(1, 600)) for _ in range(3))    # anything
        out.append((m, n, k, int(rng.integers(0, 2)), int(rng.integers(0, 2)), i))
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,lhs_t,rhs_t,seed", cases())
def test_bf16_dot_general_layouts(m, n, k, lhs_t, rhs_t, seed):
    oracle, _ = entry.load_oracle()
    rng = np.random.default_rng(seed)
    a = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))   # logical [M][K]
    b = oracle.round_to_bf16(rng.standard_normal((k, n)).astype(np.float32))   # logical [K][N]
    lhs = a.T.copy() if lhs_t else a
    rhs = b.T.copy() if rhs_t else b
    out_et = "f32" if seed % 4 == 3 else "bf16"
    text = dot_module(lhs.shape, rhs.shape, 0 if lhs_t else 1, 1 if rhs_t else 0, (m, n), "bf16", out_et)
    f = rx.compile(text)
    # host arrays cross the boundary with reversed dims
    out = f(rx.to_rarray(np.ascontiguousarray(lhs.T).astype(rx.bfloat16)), rx.to_rarray(np.ascontiguousarray(rhs.T).astype(rx.bfloat16)))
    got = np.asarray(out).T.astype(np.float64)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert got.shape == want.shape
    scale = np.abs(want).max() + 1e-30
    assert np.abs(got - want).max() / scale <= 2e-2
    if out_et == "f32":   # fp32 accumulation only
        np.testing.assert_allclose(got, want, rtol=1e-4, atol=scale * 1e-5)
    else:                 # plus the final rounding to bf16 (2^-9 relative)
        np.testing.assert_allclose(got, want, rtol=2 ** -7, atol=scale * 2 ** -8)
