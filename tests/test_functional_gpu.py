"""Activation / loss Functions, modules and Adam of the host mirror, driven like the reference's
own tests drive its Functions (forward(ctx, ...) / backward(ctx, grad_out), modules with autograd),
and held to what the reference's CPU path produced for the same inputs (tests/golden)."""
from __future__ import annotations

import numpy as np
import pytest

from _gpu_util import assert_same_bits

pytestmark = pytest.mark.gpu


def _mods():
    from keydnn_v2_b200 import Context, Parameter, Tensor
    from keydnn_v2_b200 import functional as F

    return Tensor, Parameter, Context, F


def test_functions_forward_backward_like_the_reference_tests(golden):
    Tensor, _, Context, F = _mods()
    x, go = golden["act/x"], golden["act/go"]
    tol = dict(rtol=2e-6, atol=1e-7)
    for name, fn, kw, exact in (("exp", F.ExpFn, {}, False), ("sigmoid", F.SigmoidFn, {}, False), ("relu", F.ReLUFn, {}, True),
                                ("tanh", F.TanhFn, {}, False), ("leaky", F.LeakyReLUFn, {"alpha": 0.1}, True),
                                ("softmax1", F.SoftmaxFn, {"axis": -1}, False), ("softmax0", F.SoftmaxFn, {"axis": 0}, False)):
        tx = Tensor.from_numpy(x)
        ctx = Context((tx,), None)
        y = fn.forward(ctx, tx, **kw)
        g = fn.backward(ctx, Tensor.from_numpy(go))
        g = g[0] if isinstance(g, tuple) else g
        if exact:
            assert_same_bits(y.to_numpy(), golden[f"act/{name}_y"], err_msg=name)
            assert_same_bits(g.to_numpy(), golden[f"act/{name}_gx"], err_msg=name)
        else:
            np.testing.assert_allclose(y.to_numpy(), golden[f"act/{name}_y"], err_msg=name, **tol)
            np.testing.assert_allclose(g.to_numpy(), golden[f"act/{name}_gx"], err_msg=name, rtol=1e-4, atol=1e-6)


def test_modules_attach_autograd_and_accumulate(golden):
    Tensor, _, _, F = _mods()
    x, go = golden["act/x"], golden["act/go"]
    for name, mod in (("sigmoid", F.Sigmoid()), ("relu", F.ReLU()), ("tanh", F.Tanh()), ("leaky", F.LeakyReLU(0.1)),
                      ("softmax1", F.Softmax(axis=-1)), ("softmax0", F.Softmax(axis=0))):
        tx = Tensor.from_numpy(x, requires_grad=True)
        y = mod(tx)
        assert y.requires_grad and y._ctx is not None
        y.backward(Tensor.from_numpy(go))
        np.testing.assert_allclose(tx.grad.to_numpy(), golden[f"act/{name}_gx"], rtol=1e-4, atol=1e-6, err_msg=name)
        assert y._ctx is None                            # graph released after backward
        ty = mod(Tensor.from_numpy(x))                   # outside the graph: no node
        assert not ty.requires_grad and ty._ctx is None
    with pytest.raises(ValueError):
        F.Softmax(axis=2)(Tensor.from_numpy(x))


def test_tensor_exp_log_sqrt_methods(golden):
    Tensor, _, _, _ = _mods()
    xp, go = golden["act/xpos"], golden["act/go"]
    for name, exact in (("log", False), ("sqrt", True)):
        t = Tensor.from_numpy(xp, requires_grad=True)
        y = getattr(t, name)()
        y.backward(Tensor.from_numpy(go))
        if exact:
            assert_same_bits(y.to_numpy(), golden[f"act/{name}_y"])
            assert_same_bits(t.grad.to_numpy(), golden[f"act/{name}_gx"])
        else:
            np.testing.assert_allclose(y.to_numpy(), golden[f"act/{name}_y"], rtol=2e-6, atol=1e-7)
            assert_same_bits(t.grad.to_numpy(), golden[f"act/{name}_gx"])      # g / x: no transcendental
    t = Tensor.from_numpy(golden["act/x"], requires_grad=True)
    y = t.exp()
    y.backward(Tensor.from_numpy(go))
    np.testing.assert_allclose(y.to_numpy(), golden["act/exp_y"], rtol=2e-6)
    np.testing.assert_allclose(t.grad.to_numpy(), golden["act/exp_gx"], rtol=2e-6, atol=1e-7)


def test_losses_through_autograd(golden):
    Tensor, _, _, F = _mods()
    pred = golden["loss/pred"]
    g = Tensor.full((), float(golden["loss/g"]))
    for name, fn, tgt, exact_grad in (("sse", F.sse_loss, "target", True), ("mse", F.mse_loss, "target", True),
                                      ("bce", F.binary_cross_entropy, "binary", True),
                                      ("cce", F.categorical_cross_entropy, "onehot", True)):
        tp = Tensor.from_numpy(pred, requires_grad=True)
        tt = Tensor.from_numpy(golden[f"loss/{tgt}"], requires_grad=name in ("sse", "mse"))
        loss = fn(tp, tt)
        assert loss.shape == () and loss.requires_grad
        np.testing.assert_allclose(loss.item(), golden[f"loss/{name}_y"], rtol=1e-6)
        loss.backward(g)
        assert_same_bits(tp.grad.to_numpy(), golden[f"loss/{name}_gpred"], err_msg=name)
        if name in ("sse", "mse"):
            assert_same_bits(tt.grad.to_numpy(), golden[f"loss/{name}_gtarget"], err_msg=name)
        else:
            assert tt.grad is None
    with pytest.raises(ValueError):
        F.mse_loss(Tensor.from_numpy(pred), Tensor.from_numpy(pred[:3]))


def test_unit_seed_backward_needs_no_host_read(oracle):
    """loss.backward() with the implicit gradient of one: the kernels get a null upstream pointer."""
    Tensor, _, _, F = _mods()
    rng = np.random.default_rng(2)
    pred = rng.uniform(0.1, 0.9, (8, 5)).astype(np.float32)
    onehot = np.eye(5, dtype=np.float32)[rng.integers(0, 5, 8)]
    tp = Tensor.from_numpy(pred, requires_grad=True)
    F.categorical_cross_entropy(tp, Tensor.from_numpy(onehot)).backward()
    assert_same_bits(tp.grad.to_numpy(), oracle.cce_backward(pred, onehot, 1.0))


@pytest.mark.parametrize("tag,wd", [("adam", 0.0), ("adam_wd", 1e-2)])
def test_adam_optimizer_follows_the_reference_bitwise(golden, tag, wd):
    Tensor, Parameter, _, F = _mods()
    p = Parameter.from_numpy(golden["adam/p0"])
    opt = F.Adam([p], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd)
    for k in range(3):
        opt.zero_grad()
        p.grad = Tensor.from_numpy(golden[f"adam/g{k + 1}"])
        opt.step()
        assert_same_bits(p.to_numpy(), golden[f"{tag}/p{k + 1}"])
    st = opt._state[id(p)]
    assert st["t"] == 3
    assert_same_bits(st["m"].to_numpy(), golden[f"{tag}/m3"])
    assert_same_bits(st["v"].to_numpy(), golden[f"{tag}/v3"])
    for bad in (dict(lr=0.0), dict(betas=(1.0, 0.9)), dict(eps=0.0), dict(weight_decay=-1.0)):
        with pytest.raises(ValueError):
            F.Adam([p], **bad)


def test_softmax_classifier_trains_with_adam():
    """End to end on the device: Linear -> Softmax -> CCE, Adam; the loss must fall."""
    Tensor, _, _, F = _mods()
    from keydnn_v2_b200 import nn

    np.random.seed(0)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((256, 20)).astype(np.float32)
    w_true = rng.standard_normal((20, 4)).astype(np.float32)
    labels = (x @ w_true).argmax(1)
    t = Tensor.from_numpy(np.eye(4, dtype=np.float32)[labels])
    lin = nn.Linear(20, 4)
    opt = F.Adam(lin.parameters(), lr=5e-2)
    tx = Tensor.from_numpy(x)
    losses = []
    for _ in range(40):
        opt.zero_grad()
        loss = F.categorical_cross_entropy(F.softmax(lin(tx)), t)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.35 * losses[0], losses[::8]


def test_flat_buffer_adam_equals_the_per_parameter_one(golden):
    """nn.Adam keeps all parameters in one buffer and updates them with one launch: same bits as the
    reference-pinned per-parameter optimizer; a recorded step refuses it (per-step host scalars)."""
    Tensor, Parameter, _, F = _mods()
    from keydnn_v2_b200 import nn

    rng = np.random.default_rng(4)
    extra = rng.standard_normal((7, 5)).astype(np.float32)
    ps = [Parameter.from_numpy(golden["adam/p0"]), Parameter.from_numpy(extra)]
    qs = [Parameter.from_numpy(golden["adam/p0"]), Parameter.from_numpy(extra)]
    flat = nn.Adam(ps, lr=1e-2, weight_decay=1e-2)
    each = F.Adam(qs, lr=1e-2, weight_decay=1e-2)
    for k in range(3):
        g_extra = rng.standard_normal(extra.shape).astype(np.float32)
        for group in (ps, qs):
            group[0].grad = Tensor.from_numpy(golden[f"adam/g{k + 1}"])
            group[1].grad = Tensor.from_numpy(g_extra)
        flat.step()
        each.step()
        assert_same_bits(ps[0].to_numpy(), golden[f"adam_wd/p{k + 1}"])
        for a, b in zip(ps, qs):
            assert_same_bits(a.to_numpy(), b.to_numpy())
    model = nn.Linear(4, 2)
    x = Tensor.from_numpy(rng.standard_normal((3, 4)).astype(np.float32))
    t = Tensor.from_numpy(rng.standard_normal((3, 2)).astype(np.float32))
    with pytest.raises(TypeError):
        nn.GraphedTrainStep(model, nn.Adam(model.parameters()), x, t)


def test_adam_with_the_step_count_on_the_device_same_bits_and_recordable(golden):
    """device_step=True: the bias corrections come from a table indexed by a device counter; same bits as passing
    them by value, and a training step with it can be recorded in a CUDA graph and replayed."""
    Tensor, Parameter, _, _ = _mods()
    from keydnn_v2_b200 import nn

    rng = np.random.default_rng(14)
    p0 = golden["adam/p0"]
    a, b = Parameter.from_numpy(p0), Parameter.from_numpy(p0)
    by_value = nn.Adam([a], lr=1e-2, weight_decay=1e-2)
    counted = nn.Adam([b], lr=1e-2, weight_decay=1e-2, device_step=True)
    assert counted.graph_safe and not by_value.graph_safe
    for k in range(6):
        g = golden[f"adam/g{k + 1}"] if k < 3 else (rng.standard_normal(p0.shape) * 0.1).astype(np.float32)
        a.grad, b.grad = Tensor.from_numpy(g), Tensor.from_numpy(g)
        by_value.step()
        counted.step()
        assert_same_bits(b.to_numpy(), a.to_numpy())
        if k < 3:
            assert_same_bits(b.to_numpy(), golden[f"adam_wd/p{k + 1}"])
    # recorded: Linear -> MSE with Adam, replays against eager steps of a twin
    x = Tensor.from_numpy(rng.standard_normal((32, 12)).astype(np.float32))
    t = Tensor.from_numpy(rng.standard_normal((32, 3)).astype(np.float32))
    losses = {}
    for mode in ("eager", "graph"):
        np.random.seed(9)
        model = nn.Linear(12, 3)
        opt = nn.Adam(model.parameters(), lr=5e-2, device_step=True)
        if mode == "eager":
            losses[mode] = [nn.train_step(model, opt, x, t).item() for _ in range(7)]
        else:
            g = nn.GraphedTrainStep(model, opt, x, t, warmup=2)
            try:
                losses[mode] = [g.run().item() for _ in range(5)]
            finally:
                g.close()
    np.testing.assert_allclose(losses["graph"], losses["eager"][2:7], rtol=1e-5)
    assert losses["eager"][-1] < losses["eager"][0]
