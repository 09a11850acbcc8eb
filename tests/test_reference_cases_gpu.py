"""Cases the reference's own test-suite checks for activations, losses and optimizers
(tests/infrastructure/test_function.py, test_activations.py, test_losses.py, test_optimizers.py, test_exp.py),
restated against the CUDA mirror: closed forms, finite differences, scaling with the upstream gradient,
optimizer bookkeeping and argument errors."""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _kd():
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import functional as F
    from keydnn_v2_b200 import nn

    return kd, F, nn


def _numeric_grad(f, x: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    g = np.zeros_like(x)
    flat, gf = x.reshape(-1), g.reshape(-1)
    for i in range(flat.size):
        old = flat[i]
        flat[i] = old + eps
        up = f(x)
        flat[i] = old - eps
        down = f(x)
        flat[i] = old
        gf[i] = (up - down) / (2 * eps)
    return g


@pytest.mark.parametrize("name", ["sigmoid", "tanh", "leaky_relu", "relu", "exp", "log", "sqrt"])
def test_activation_backward_matches_finite_differences_in_fp64(name):
    kd, F, _ = _kd()
    rng = np.random.default_rng(5)
    x = rng.uniform(0.3, 2.0, (3, 4)) if name in ("log", "sqrt") else rng.uniform(-2, 2, (3, 4))
    x[np.abs(x) < 0.05] = 0.5                                     # keep away from the kinks of relu / leaky relu
    w = rng.standard_normal(x.shape)
    fn = getattr(F, name)

    def scalar(arr):
        return float((fn(kd.Tensor.from_numpy(arr)).to_numpy() * w).sum())

    tx = kd.Tensor.from_numpy(x.copy(), requires_grad=True)
    fn(tx).backward(kd.Tensor.from_numpy(w))
    np.testing.assert_allclose(tx.grad.to_numpy(), _numeric_grad(scalar, x.copy()), rtol=1e-6, atol=1e-8)


def test_closed_forms_of_the_activation_functions():
    kd, F, _ = _kd()
    x = np.array([[-2.0, -0.5, 0.0, 0.5, 3.0]], np.float32)
    t = kd.Tensor.from_numpy(x)
    np.testing.assert_array_equal(F.relu(t).to_numpy(), np.maximum(x, 0))
    np.testing.assert_allclose(F.leaky_relu(t).to_numpy(), np.where(x > 0, x, 0.01 * x), rtol=1e-6)       # default alpha
    np.testing.assert_allclose(F.leaky_relu(t, 0.2).to_numpy(), np.where(x > 0, x, 0.2 * x), rtol=1e-6)
    np.testing.assert_allclose(F.sigmoid(t).to_numpy(), 1 / (1 + np.exp(-x)), rtol=1e-6)
    np.testing.assert_allclose(F.tanh(t).to_numpy(), np.tanh(x), rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(F.exp(t).to_numpy(), np.exp(x), rtol=1e-6)
    g = np.array([[1.0, 2.0, 3.0, 4.0, 5.0]], np.float32)
    tx = kd.Tensor.from_numpy(x, requires_grad=True)
    F.relu(tx).backward(kd.Tensor.from_numpy(g))
    np.testing.assert_array_equal(tx.grad.to_numpy(), g * (x > 0))
    y = F.sigmoid(kd.Tensor.from_numpy(x)).to_numpy()
    tx = kd.Tensor.from_numpy(x, requires_grad=True)
    F.sigmoid(tx).backward(kd.Tensor.from_numpy(g))
    np.testing.assert_allclose(tx.grad.to_numpy(), g * y * (1 - y), rtol=1e-5)
    # exp: gradient is grad_out * out; nothing is attached outside the graph
    tx = kd.Tensor.from_numpy(x, requires_grad=True)
    out = F.exp(tx)
    assert out.requires_grad and out._ctx is not None and F.exp(kd.Tensor.from_numpy(x))._ctx is None
    out.backward(kd.Tensor.from_numpy(g))
    np.testing.assert_allclose(tx.grad.to_numpy(), g * np.exp(x), rtol=1e-6)
    with pytest.raises((TypeError, AttributeError)):
        F.exp(x)                                                   # a NumPy array is not a Tensor


def test_softmax_rows_sum_to_one_jvp_and_finite_differences():
    kd, F, _ = _kd()
    rng = np.random.default_rng(8)
    x = rng.standard_normal((4, 6))
    g = rng.standard_normal((4, 6))
    tx = kd.Tensor.from_numpy(x.copy(), requires_grad=True)
    y = F.softmax(tx, axis=-1)
    yv = y.to_numpy()
    np.testing.assert_allclose(yv.sum(1), 1.0, rtol=1e-12)
    y.backward(kd.Tensor.from_numpy(g))
    np.testing.assert_allclose(tx.grad.to_numpy(), yv * (g - (g * yv).sum(1, keepdims=True)), rtol=1e-10, atol=1e-14)

    def scalar(arr):
        return float((F.softmax(kd.Tensor.from_numpy(arr), axis=-1).to_numpy() * g).sum())

    np.testing.assert_allclose(tx.grad.to_numpy(), _numeric_grad(scalar, x.copy()), rtol=1e-5, atol=1e-8)
    for bad in (2, -3):
        with pytest.raises(ValueError):
            F.softmax(kd.Tensor.from_numpy(x), axis=bad)


@pytest.mark.parametrize("name", ["sse", "mse", "bce", "cce"])
def test_loss_values_gradients_and_scaling_with_the_upstream_gradient(name):
    kd, F, _ = _kd()
    rng = np.random.default_rng(3)
    pred = rng.uniform(0.1, 0.9, (5, 4))
    if name == "cce":
        pred /= pred.sum(1, keepdims=True)
        target = np.eye(4)[rng.integers(0, 4, 5)]
    elif name == "bce":
        target = (rng.uniform(size=pred.shape) > 0.5).astype(np.float64)
    else:
        target = rng.standard_normal(pred.shape)
    fn = {"sse": F.sse_loss, "mse": F.mse_loss, "bce": F.binary_cross_entropy, "cce": F.categorical_cross_entropy}[name]
    want = {"sse": lambda p: ((p - target) ** 2).sum(), "mse": lambda p: ((p - target) ** 2).mean(),
            "bce": lambda p: -(target * np.log(p) + (1 - target) * np.log(1 - p)).mean(),
            "cce": lambda p: -(target * np.log(p)).sum() / p.shape[0]}[name]
    tt = kd.Tensor.from_numpy(target)

    def value(arr):
        return fn(kd.Tensor.from_numpy(arr), tt).item()

    np.testing.assert_allclose(value(pred), want(pred), rtol=1e-12)
    grads = []
    for scale in (1.0, 2.5):
        tp = kd.Tensor.from_numpy(pred.copy(), requires_grad=True)
        fn(tp, tt).backward(kd.Tensor.full((), scale, np.float64))
        grads.append(tp.grad.to_numpy())
    np.testing.assert_allclose(grads[1], 2.5 * grads[0], rtol=1e-12)                      # scales with grad_out
    np.testing.assert_allclose(grads[0], _numeric_grad(value, pred.copy(), 1e-7), rtol=1e-5, atol=1e-7)
    with pytest.raises(ValueError):
        fn(kd.Tensor.from_numpy(pred), kd.Tensor.from_numpy(target[:2]))


@pytest.mark.parametrize("which", ["sgd", "adam"])
def test_optimizer_bookkeeping_like_the_reference(which):
    kd, F, nn = _kd()
    rng = np.random.default_rng(1)
    a0, b0 = rng.standard_normal(6).astype(np.float32), rng.standard_normal((2, 3)).astype(np.float32)
    make = (lambda ps, **kw: nn.SGD(ps, lr=0.1, **kw)) if which == "sgd" else (lambda ps, **kw: nn.Adam(ps, lr=0.1, **kw))
    # a parameter without a gradient is skipped entirely, weight decay included
    a, b = kd.Parameter.from_numpy(a0), kd.Parameter.from_numpy(b0)
    opt = make([a, b], weight_decay=0.5)
    a.grad = kd.Tensor.from_numpy(np.ones(6, np.float32))
    opt.step()
    np.testing.assert_array_equal(b.to_numpy(), b0)
    assert not np.array_equal(a.to_numpy(), a0)
    if which == "sgd":
        np.testing.assert_allclose(a.to_numpy(), a0 - 0.1 * (1.0 + 0.5 * a0), rtol=1e-6)      # g + wd * p
    else:
        g_eff = 1.0 + 0.5 * a0                                                               # first step: m_hat = g, v_hat = g^2
        np.testing.assert_allclose(a.to_numpy(), a0 - 0.1 * g_eff / (np.abs(g_eff) + 1e-8), rtol=1e-5)
    opt.zero_grad()
    assert a.grad is None and b.grad is None
    opt.step()                                                                               # nothing has a gradient: no-op
    np.testing.assert_array_equal(b.to_numpy(), b0)
    # weight decay changes the update
    outs = []
    for wd in (0.0, 0.3):
        p = kd.Parameter.from_numpy(a0)
        o = make([p], weight_decay=wd)
        p.grad = kd.Tensor.from_numpy(np.full(6, 0.2, np.float32))
        o.step()
        outs.append(p.to_numpy())
    assert not np.allclose(outs[0], outs[1])
    bad = [dict(lr=0.0), dict(weight_decay=-0.1)] + ([dict(betas=(0.0, 0.9)), dict(betas=(0.9, 1.0)), dict(eps=0.0)] if which == "adam" else [])
    for kw in bad:
        with pytest.raises(ValueError):
            (nn.SGD if which == "sgd" else nn.Adam)([kd.Parameter.from_numpy(a0)], **kw)
