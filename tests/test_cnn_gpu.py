"""One training step of the small CNN on the GPU against the same step run by the reference itself
on its CPU path (tests/golden/, `cnn/*`): forward, MSE loss, every parameter gradient, SGD update.
Conv / Linear go through cuDNN / cuBLAS as in the reference; BatchNorm2d, ReLU, pooling, loss and the
optimizer go through this library's kernels."""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _model(kd, nn, golden, dtype):
    np.random.seed(0)
    model = nn.Sequential(
        nn.Conv2d(3, 4, 3, padding=1, dtype=dtype), nn.BatchNorm2d(4, dtype=dtype), nn.ReLU(), nn.MaxPool2d(2),
        nn.Conv2d(4, 6, 3, padding=1, dtype=dtype), nn.BatchNorm2d(6, dtype=dtype), nn.ReLU(), nn.GlobalAvgPool2d(),
        nn.Flatten(), nn.Linear(6, 3, dtype=dtype),
    )
    params = model.parameters()
    assert len(params) == int(golden["cnn/n_params"][0])
    for i, p in enumerate(params):
        init = golden[f"cnn/p{i}_init"]
        assert p.shape == init.shape
        p.copy_from_numpy(init.astype(dtype))
    return model, params


@pytest.mark.parametrize("dtype,tol", [(np.float32, dict(rtol=5e-3, atol=5e-4)), (np.float64, dict(rtol=2e-4, atol=2e-5))])
def test_training_step_matches_the_reference_cpu_step(golden, dtype, tol):
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    if dtype == np.float64:
        nn.ReLU.forward = _relu_any_dtype            # the mask kernels write float32; f64 check casts it
    model, params = _model(kd, nn, golden, dtype)
    opt = nn.SGD(params, lr=0.01, weight_decay=1e-4)
    x = kd.Tensor.from_numpy(golden["cnn/x"].astype(dtype))
    t = kd.Tensor.from_numpy(golden["cnn/t"].astype(dtype))
    opt.zero_grad()
    pred = model(x)
    loss = nn.mse_loss(pred, t)
    loss.backward()
    np.testing.assert_allclose(pred.to_numpy(), golden["cnn/pred"], **tol)
    np.testing.assert_allclose(loss.to_numpy(), golden["cnn/loss"].reshape(()), **tol)
    for i, p in enumerate(params):
        assert p.grad is not None, i
        np.testing.assert_allclose(p.grad.to_numpy(), golden[f"cnn/p{i}_grad"], err_msg=f"grad {i}", **tol)
    opt.step()
    for i, p in enumerate(params):
        np.testing.assert_allclose(p.to_numpy(), golden[f"cnn/p{i}_after"], err_msg=f"param {i}", **tol)


def _relu_any_dtype(self, x):
    """float64 variant for the check above: same mask-and-multiply, mask converted to the input type on the host."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200.tensor import Context, no_grad

    with no_grad():
        mask = kd.Tensor.from_numpy((x > 0.0).to_numpy().astype(x.dtype))
        y = x * mask
    if x._needs_grad():
        y.requires_grad = True
        y._ctx = Context((x,), lambda g: (_nograd_mul(g, mask),))
    return y


def _nograd_mul(a, b):
    from keydnn_v2_b200.tensor import no_grad

    with no_grad():
        return a * b


def test_batchnorm_eval_mode_and_running_stats():
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    rng = np.random.default_rng(2)
    x = rng.standard_normal((8, 5, 6, 6)).astype(np.float32) * 2 + 1
    bn = nn.BatchNorm2d(5)
    y = bn(kd.Tensor.from_numpy(x))
    mu, var = x.mean((0, 2, 3)), x.var((0, 2, 3))
    np.testing.assert_allclose(y.to_numpy(), (x - mu[None, :, None, None]) / np.sqrt(var + 1e-5)[None, :, None, None],
                               rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(bn.running_mean.to_numpy(), 0.1 * mu, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(bn.running_var.to_numpy(), 0.9 + 0.1 * var, rtol=1e-5, atol=1e-6)
    bn.eval()
    y2 = bn(kd.Tensor.from_numpy(x)).to_numpy()
    rm, rv = bn.running_mean.to_numpy(), bn.running_var.to_numpy()
    np.testing.assert_allclose(y2, (x - rm[None, :, None, None]) / np.sqrt(rv + 1e-5)[None, :, None, None], rtol=1e-4,
                               atol=1e-5)


def test_momentum_training_reduces_the_loss():
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    np.random.seed(3)
    rng = np.random.default_rng(3)
    model = nn.small_cnn()
    opt = nn.SGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    x = kd.Tensor.from_numpy(rng.standard_normal((32, 3, 64, 64)).astype(np.float32))
    t = kd.Tensor.from_numpy(np.eye(10, dtype=np.float32)[rng.integers(0, 10, 32)])
    losses = [nn.train_step(model, opt, x, t).item() for _ in range(15)]
    assert np.isfinite(losses).all() and losses[-1] < 0.7 * losses[0], losses


def test_fused_batchnorm_relu_is_bit_identical_to_the_two_layers():
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    rng = np.random.default_rng(6)
    x = rng.standard_normal((6, 5, 8, 12)).astype(np.float32)
    g = rng.standard_normal(x.shape).astype(np.float32)
    outs = []
    for fuse in (True, False):
        np.random.seed(0)
        bn = nn.BatchNorm2d(5)
        bn.gamma.copy_from_numpy(np.linspace(-1, 1.5, 5).astype(np.float32))
        bn.beta.copy_from_numpy(np.linspace(0.3, -0.3, 5).astype(np.float32))
        seq = nn.Sequential(bn, nn.ReLU(), fuse=fuse)
        assert bn.fused_relu == fuse
        tx = kd.Tensor.from_numpy(x, requires_grad=True)
        y = seq(tx)
        y.backward(kd.Tensor.from_numpy(g))
        outs.append((y.to_numpy(), tx.grad.to_numpy(), bn.gamma.grad.to_numpy(), bn.beta.grad.to_numpy()))
    for a, b in zip(*outs):
        np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("training", [True, False])
def test_conv_bias_added_by_batchnorm_is_bit_identical_to_the_bias_pass(training):
    """Conv2d -> BatchNorm2d -> ReLU with the convolution's bias added inside the BatchNorm kernels, against the same
    stack with a separate bias pass: outputs, running statistics and every gradient must have the same bits."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    rng = np.random.default_rng(16)
    x = rng.standard_normal((5, 3, 10, 12)).astype(np.float32)
    g = rng.standard_normal((5, 6, 10, 12)).astype(np.float32)
    bias = rng.standard_normal(6).astype(np.float32)
    outs = []
    for fuse in (True, False):
        np.random.seed(2)
        conv, bn = nn.Conv2d(3, 6, 3, padding=1), nn.BatchNorm2d(6)
        conv.bias.copy_from_numpy(bias)
        bn.gamma.copy_from_numpy(np.linspace(0.5, 1.5, 6).astype(np.float32))
        bn.beta.copy_from_numpy(np.linspace(0.2, -0.2, 6).astype(np.float32))
        seq = nn.Sequential(conv, bn, nn.ReLU(), fuse=fuse)
        assert conv.bias_deferred == fuse and (bn.pre_bias is conv.bias) == fuse
        seq.train(training)
        tx = kd.Tensor.from_numpy(x, requires_grad=True)
        y = seq(tx)
        y.backward(kd.Tensor.from_numpy(g))
        outs.append((y.to_numpy(), tx.grad.to_numpy(), conv.weight.grad.to_numpy(), conv.bias.grad.to_numpy(),
                     bn.gamma.grad.to_numpy(), bn.beta.grad.to_numpy(), bn.running_mean.to_numpy(), bn.running_var.to_numpy()))
    for i, (a, b) in enumerate(zip(*outs)):
        if i in (1, 2):      # input / weight gradients come from cuDNN, whose reduction order is its own
            np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)
        else:
            np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32), err_msg=str(i))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape,relu", [((5, 6, 8, 16), True), ((3, 4, 12, 24), False), ((2, 3, 10, 12), True)])
def test_batchnorm_relu_maxpool_in_one_pass_is_bit_identical_to_the_layers(shape, relu, dtype):
    """BatchNorm2d (+ ReLU) -> MaxPool2d(2) computed by the BatchNorm kernels (the normalised activation and its
    gradient are never stored) against the separate layers; the last shape (W % 8 != 0) takes the fallback."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    N, C, H, W = shape
    rng = np.random.default_rng(H * W)
    x = rng.standard_normal(shape).astype(dtype)
    x = (np.round(x * 4) / 4).astype(dtype)                      # ties inside windows: the first position must win
    g = rng.standard_normal((N, C, H // 2, W // 2)).astype(dtype)
    outs = []
    for fuse in (True, False):
        bn = nn.BatchNorm2d(C, dtype=dtype)
        bn.gamma.copy_from_numpy(np.linspace(-1.0, 1.5, C).astype(dtype))
        bn.beta.copy_from_numpy(np.linspace(0.3, -0.3, C).astype(dtype))
        layers = [bn] + ([nn.ReLU()] if relu else []) + [nn.MaxPool2d(2)]
        seq = nn.Sequential(*layers, fuse=fuse)
        assert (bn.fused_pool is not None) == fuse
        tx = kd.Tensor.from_numpy(x, requires_grad=True)
        y = seq(tx)
        assert y.shape == (N, C, H // 2, W // 2)
        y.backward(kd.Tensor.from_numpy(g))
        outs.append((y.to_numpy(), tx.grad.to_numpy(), bn.gamma.grad.to_numpy(), bn.beta.grad.to_numpy(),
                     bn.running_mean.to_numpy(), bn.running_var.to_numpy()))
    view = np.uint32 if dtype == np.float32 else np.uint64
    for i, (a, b) in enumerate(zip(*outs)):
        np.testing.assert_array_equal(a.view(view), b.view(view), err_msg=str(i))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape,relu", [((6, 5, 16, 16), True), ((3, 4, 10, 12), False), ((2, 3, 6, 6), True)])
def test_batchnorm_relu_global_avgpool_in_one_pass_is_bit_identical_to_the_layers(shape, relu, dtype):
    """BatchNorm2d (+ ReLU) -> GlobalAvgPool2d computed by the BatchNorm kernels against the separate layers; the
    last shape (HW <= 64) takes the fallback."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    N, C, H, W = shape
    rng = np.random.default_rng(H + W)
    x = rng.standard_normal(shape).astype(dtype)
    g = rng.standard_normal((N, C, 1, 1)).astype(dtype)
    outs = []
    for fuse in (True, False):
        bn = nn.BatchNorm2d(C, dtype=dtype)
        bn.gamma.copy_from_numpy(np.linspace(-1.0, 1.5, C).astype(dtype))
        bn.beta.copy_from_numpy(np.linspace(0.3, -0.3, C).astype(dtype))
        layers = [bn] + ([nn.ReLU()] if relu else []) + [nn.GlobalAvgPool2d()]
        seq = nn.Sequential(*layers, fuse=fuse)
        assert (bn.fused_gap is not None) == fuse
        tx = kd.Tensor.from_numpy(x, requires_grad=True)
        y = seq(tx)
        assert y.shape == (N, C, 1, 1)
        y.backward(kd.Tensor.from_numpy(g))
        outs.append((y.to_numpy(), tx.grad.to_numpy(), bn.gamma.grad.to_numpy(), bn.beta.grad.to_numpy(),
                     bn.running_mean.to_numpy(), bn.running_var.to_numpy()))
    view = np.uint32 if dtype == np.float32 else np.uint64
    for i, (a, b) in enumerate(zip(*outs)):
        np.testing.assert_array_equal(a.view(view), b.view(view), err_msg=str(i))


def test_graphed_training_step_follows_the_eager_one():
    """A CUDA-graph replay of the step must train exactly like the eager step sequence."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    rng = np.random.default_rng(11)
    hx = rng.standard_normal((16, 3, 32, 32)).astype(np.float32)
    ht = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 16)]
    losses = {}
    for mode in ("eager", "graph"):
        np.random.seed(7)
        model = nn.small_cnn()
        opt = nn.SGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
        x, t = kd.Tensor.from_numpy(hx), kd.Tensor.from_numpy(ht)
        if mode == "eager":
            losses[mode] = [nn.train_step(model, opt, x, t).item() for _ in range(8)]
        else:
            g = nn.GraphedTrainStep(model, opt, x, t, warmup=3)       # 3 eager + 1 recorded (not executed) step
            try:
                seq = [g.run().item() for _ in range(5)]
            finally:
                g.close()
            losses[mode] = seq
            after = nn.train_step(model, opt, x, t).item()            # eager again after the graph is gone
            assert np.isfinite(after)
    # graph replays 1..5 correspond to eager steps 4..8 (three warm-up steps came first)
    np.testing.assert_allclose(losses["graph"], losses["eager"][3:8], rtol=2e-3, atol=1e-5)
    assert losses["eager"][-1] < losses["eager"][0]


def test_training_off_the_default_stream_equals_training_on_it():
    """Five eager training steps with the library moved to a created non-blocking stream: Conv2d / Linear (cuDNN /
    cuBLAS, second library) must follow the BatchNorm / pooling / loss / optimizer kernels onto that stream.  A
    library left on the legacy stream races with them (a non-blocking stream does not synchronise with it) and the
    losses come out different or NaN.  Tolerance 1e-5: cuDNN's weight-gradient algorithm may add in any order."""
    import ctypes

    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn
    from keydnn_v2_b200._native import load_dnn

    lib, dnn = kd.load(), load_dnn()
    rng = np.random.default_rng(21)
    hx = rng.standard_normal((64, 3, 64, 64)).astype(np.float32)
    ht = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 64)]
    prev, stream, seen = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_uint64(0)
    lib.call("keydnn_cuda_get_stream", ctypes.byref(prev))
    lib.call("keydnn_cuda_stream_create", ctypes.byref(stream))
    runs = {}
    try:
        for where in ("default", "created"):
            lib.call("keydnn_cuda_synchronize")
            lib.call("keydnn_cuda_set_stream", prev.value if where == "default" else stream.value)
            dnn.call("keydnn_dnn_get_stream", ctypes.byref(seen))
            assert seen.value == (prev.value if where == "default" else stream.value)
            np.random.seed(5)
            model = nn.small_cnn()
            opt = nn.SGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
            x, t = kd.Tensor.from_numpy(hx), kd.Tensor.from_numpy(ht)
            losses = [nn.train_step(model, opt, x, t) for _ in range(5)]      # no host read between the steps
            runs[where] = ([v.item() for v in losses], [p.to_numpy() for p in model.parameters()])
    finally:
        lib.call("keydnn_cuda_synchronize")
        lib.call("keydnn_cuda_set_stream", prev.value)
        lib.call("keydnn_cuda_stream_destroy", stream.value)
    assert np.all(np.isfinite(runs["created"][0]))
    np.testing.assert_allclose(runs["created"][0], runs["default"][0], rtol=1e-5)
    for a, b in zip(runs["created"][1], runs["default"][1]):
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)
    assert runs["default"][0][-1] < runs["default"][0][0]


def test_pipelined_feeding_trains_on_the_batches_it_is_given():
    """step_async / loss_of: two alternating batches fed from pinned host memory through the staging
    buffers must give the losses of the same sequence run with plain copies and graph launches."""
    import ctypes

    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    lib = kd.load()
    rng = np.random.default_rng(12)

    def pinned(a):
        p = ctypes.c_void_p(0)
        lib.call("keydnn_cuda_host_alloc", ctypes.byref(p), a.nbytes)
        out = np.frombuffer((ctypes.c_char * a.nbytes).from_address(p.value), dtype=a.dtype).reshape(a.shape)
        out[...] = a
        return out, p

    batches = []
    for _ in range(2):
        hx, px = pinned(rng.standard_normal((16, 3, 32, 32)).astype(np.float32))
        ht, pt = pinned(np.eye(10, dtype=np.float32)[rng.integers(0, 10, 16)])
        batches.append((hx, ht, px, pt))
    losses = {}
    for mode in ("plain", "pipelined"):
        np.random.seed(3)
        model = nn.small_cnn()
        opt = nn.SGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
        x, t = kd.Tensor.from_numpy(batches[0][0]), kd.Tensor.from_numpy(batches[0][1])
        g = nn.GraphedTrainStep(model, opt, x, t, warmup=2)
        try:
            seq = []
            if mode == "plain":
                for i in range(6):
                    x.copy_from_numpy(batches[i % 2][0])
                    t.copy_from_numpy(batches[i % 2][1])
                    seq.append(g.run().item())
            else:
                tickets = []
                for i in range(6):
                    tickets.append(g.step_async(batches[i % 2][0], batches[i % 2][1]))
                    if i >= 1:
                        seq.append(g.loss_of(tickets[i - 1]))
                seq.append(g.loss_of(tickets[-1]))
        finally:
            g.close()
        losses[mode] = seq
    # same batches in the same order; the convolution's weight-gradient algorithm is free to add in any order
    np.testing.assert_allclose(losses["pipelined"], losses["plain"], rtol=1e-5)
    for _, _, px, pt in batches:
        lib.call("keydnn_cuda_host_free", px)
        lib.call("keydnn_cuda_host_free", pt)
