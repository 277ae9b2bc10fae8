"""The reverse program of the MLP benchmark step is written out by hand (Enzyme's pass cannot run here), and
the engine is only ever compared with the oracle interpreting that same text.  This checks the derivation itself:
the oracle's gradients of the module must equal torch.autograd's gradients of the forward function (float64, no
bf16 rounding on either side) and a central finite difference."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")


def _forward(W1, b1, W2, b2, X, Y):
    """The primal the module differentiates: two dense layers, gelu (tanh form), mean squared error."""
    z1 = X @ W1 + b1
    c = np.sqrt(2.0 / np.pi)
    h = 0.5 * z1 * (1.0 + torch.tanh(c * (z1 + 0.044715 * z1 ** 3)))
    z2 = h @ W2 + b2
    return ((z2 - Y) ** 2).mean()


def test_hand_derived_mlp_gradients_match_autograd_and_finite_differences(rx, ref):
    F, H, O, B = 24, 40, 16, 32
    rng = np.random.default_rng(0)
    W1 = rng.standard_normal((F, H)) / np.sqrt(F)
    W2 = rng.standard_normal((H, O)) / np.sqrt(H)
    b1, b2 = 0.1 * rng.standard_normal(H), 0.1 * rng.standard_normal(O)
    X, Y = rng.standard_normal((B, F)), rng.standard_normal((B, O))
    # the module with every tensor in f64, so that neither side rounds to bf16
    text = rx.programs.mlp_grad(F, H, O, B).replace("bf16", "f64").replace("xf32", "xf64").replace("tensor<f32>", "tensor<f64>")
    dW1, db1, dW2, db2, loss = ref.run_module(text, [W1, b1, W2, b2, X, Y])
    t = [torch.tensor(a, dtype=torch.float64, requires_grad=k < 4) for k, a in enumerate((W1, b1, W2, b2, X, Y))]
    L = _forward(*t)
    L.backward()
    np.testing.assert_allclose(loss, L.item(), rtol=1e-12)
    for got, want in zip((dW1, db1, dW2, db2), (t[0].grad, t[1].grad, t[2].grad, t[3].grad)):
        np.testing.assert_allclose(got, want.numpy(), rtol=1e-9, atol=1e-12)
    # central difference on a few entries of W1
    eps = 1e-6
    for (i, j) in [(0, 0), (5, 7), (23, 39)]:
        Wp, Wm = W1.copy(), W1.copy()
        Wp[i, j] += eps
        Wm[i, j] -= eps
        fd = (ref.run_module(text, [Wp, b1, W2, b2, X, Y])[4] - ref.run_module(text, [Wm, b1, W2, b2, X, Y])[4]) / (2 * eps)
        assert abs(fd - dW1[i, j]) <= 1e-6 * max(1.0, abs(dW1[i, j]))
