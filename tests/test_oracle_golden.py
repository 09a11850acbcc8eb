"""The CPU oracle against outputs of the reference itself (tests/golden/).

Pins the checker before it is trusted on the GPU: every pooling / elementwise /
reduction / optimizer function of ``oracle/`` must reproduce what the reference's
own NumPy path and C++ kernels produced for the same seeded inputs.
"""
from __future__ import annotations

import numpy as np
import pytest

POOL = {
    "k2s2p0": (2, 2, 0),
    "k3s2p1": (3, 2, 1),
    "k3s1p1": (3, 1, 1),
    "k2s2p0_odd": (2, 2, 0),
    "k23s21p10": ((2, 3), (2, 1), (1, 0)),
}


@pytest.mark.parametrize("name", sorted(POOL))
def test_maxpool_matches_reference_cpu(golden, oracle, name):
    k, s, p = POOL[name]
    x = golden[f"pool/{name}/x"]
    y, idx = oracle.maxpool2d_forward(x, k, s, p)
    np.testing.assert_array_equal(y, golden[f"pool/{name}/max_y"])
    np.testing.assert_array_equal(idx, golden[f"pool/{name}/max_idx"])
    gx = oracle.maxpool2d_backward(golden[f"pool/{name}/max_go"], idx, x.shape, p)
    # overlapping windows add in a different order in the NumPy path
    np.testing.assert_allclose(gx, golden[f"pool/{name}/max_gx"], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("name", sorted(POOL))
def test_avgpool_matches_reference_cpu(golden, oracle, name):
    k, s, p = POOL[name]
    x = golden[f"pool/{name}/x"]
    y = oracle.avgpool2d_forward(x, k, s, p)
    np.testing.assert_allclose(y, golden[f"pool/{name}/avg_y"], rtol=1e-6, atol=1e-7)
    gx = oracle.avgpool2d_backward(golden[f"pool/{name}/avg_go"], x.shape, k, s, p)
    np.testing.assert_allclose(gx, golden[f"pool/{name}/avg_gx"], rtol=1e-6, atol=1e-7)


def test_maxpool_ties_first_index(golden, oracle):
    x = golden["pool/ties/x"]
    y, idx = oracle.maxpool2d_forward(x, 2, 2, 0)
    np.testing.assert_array_equal(y, golden["pool/ties/max_y"])
    np.testing.assert_array_equal(idx, golden["pool/ties/max_idx"])
    gx = oracle.maxpool2d_backward(np.ones_like(y), idx, x.shape, 0)
    np.testing.assert_array_equal(gx, golden["pool/ties/max_gx"])


@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_pool_matches_reference_cpp_kernels_bitwise(golden, oracle, tag):
    """The reference's C++ kernels share the CUDA kernels' arithmetic: bit-exact."""
    N, C, H, W, k, s, p = (int(v) for v in golden["native/geom"])
    x = golden[f"native/{tag}/x"]
    y, idx = oracle.maxpool2d_forward(x, k, s, p)
    np.testing.assert_array_equal(y, golden[f"native/{tag}/max_y"])
    np.testing.assert_array_equal(idx, golden[f"native/{tag}/max_idx"])
    gx = oracle.maxpool2d_backward(golden[f"native/{tag}/max_go"], idx, x.shape, p)
    np.testing.assert_array_equal(gx, golden[f"native/{tag}/max_gx"])
    ya = oracle.avgpool2d_forward(x, k, s, p)
    np.testing.assert_array_equal(ya, golden[f"native/{tag}/avg_y"])
    # the C++ backward scatters go/denom per window; same terms, other order
    gxa = oracle.avgpool2d_backward(golden[f"native/{tag}/avg_go"], x.shape, k, s, p)
    tol = dict(rtol=1e-6, atol=1e-7) if tag == "f32" else dict(rtol=1e-14, atol=1e-15)
    np.testing.assert_allclose(gxa, golden[f"native/{tag}/avg_gx"], **tol)


def test_global_avgpool_matches_reference_cpu(golden, oracle):
    x = golden["gap/x"]
    np.testing.assert_allclose(oracle.global_avgpool2d_forward(x), golden["gap/y"], rtol=1e-6, atol=1e-7)
    gx = oracle.global_avgpool2d_backward(golden["gap/go"], x.shape)
    np.testing.assert_allclose(gx, golden["gap/gx"], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_arithmetic_and_backward_match_reference_cpu(golden, oracle, op):
    a, b, g = golden["ew/a"], golden["ew/b"], golden["ew/g"]
    np.testing.assert_array_equal(oracle.binary(op, a, b), golden[f"ew/{op}_y"])
    if op == "add":
        ga, gb = oracle.add_backward(g)
    elif op == "sub":
        ga, gb = oracle.sub_backward(g)
    elif op == "mul":
        ga, gb = oracle.mul_backward(g, a, b)
    else:
        ga, gb = oracle.div_backward(g, a, b)
    np.testing.assert_allclose(ga, golden[f"ew/{op}_ga"], rtol=1e-6, atol=0)
    np.testing.assert_allclose(gb, golden[f"ew/{op}_gb"], rtol=1e-6, atol=0)


def test_neg_compare_scalar_match_reference_cpu(golden, oracle):
    a = golden["ew/a"]
    np.testing.assert_array_equal(oracle.neg(a), golden["ew/neg_y"])
    np.testing.assert_array_equal(oracle.neg(golden["ew/g"]), golden["ew/neg_ga"])
    a2, b2 = golden["ew/a2"], golden["ew/b2"]
    for op in ("gt", "ge", "lt", "le"):
        out = oracle.binary(op, a2, b2)
        assert out.dtype == np.float32
        np.testing.assert_array_equal(out, golden[f"ew/{op}_y"])
    np.testing.assert_array_equal(oracle.scalar("gt", a, 0.0), golden["ew/gt_scalar_y"])
    np.testing.assert_array_equal(oracle.scalar("add", a, 1.5), golden["ew/add_scalar_y"])
    np.testing.assert_array_equal(oracle.scalar("mul", a, 0.3), golden["ew/mul_scalar_y"])
    np.testing.assert_array_equal(oracle.scalar("div", a, 0.7), golden["ew/div_scalar_y"])
    np.testing.assert_array_equal(oracle.scalar("sub", a, 0.25), golden["ew/sub_scalar_y"])


def test_reductions_match_reference_cpu(golden, oracle):
    x = golden["red/x"]
    np.testing.assert_allclose(oracle.sum_all(x), golden["red/sum_all_y"], rtol=1e-6)
    np.testing.assert_array_equal(oracle.sum_backward_fill(np.ones(1, np.float32), x.size).reshape(x.shape),
                                  golden["red/sum_all_gx"])
    np.testing.assert_allclose(oracle.mean_all(x), golden["red/mean_all_y"], rtol=1e-6)
    np.testing.assert_allclose(oracle.mean_backward_fill(np.ones(1, np.float32), x.size).reshape(x.shape),
                               golden["red/mean_all_gx"], rtol=1e-7)
    rows, cols = x.shape
    for axis in (0, 1):
        np.testing.assert_allclose(oracle.sum_axis2d(x, axis), golden[f"red/sum_axis{axis}_y"], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(oracle.sum_axis2d_serial(x, axis), golden[f"red/sum_axis{axis}_y"], rtol=1e-6,
                                   atol=1e-6)
        go = golden[f"red/sum_axis{axis}_go"]
        np.testing.assert_array_equal(oracle.sum_axis2d_backward(go, rows, cols, axis), golden[f"red/sum_axis{axis}_gx"])
        val, idx = oracle.max_axis2d(x, axis)
        np.testing.assert_array_equal(val, golden[f"red/max_axis{axis}_y"])
        go = golden[f"red/max_axis{axis}_go"]
        # no ties in this input, so the CPU path's equality mask equals the CUDA path's argmax scatter
        np.testing.assert_array_equal(oracle.max_axis2d_backward(go, idx, rows, cols, axis),
                                      golden[f"red/max_axis{axis}_gx"])


def test_sgd_matches_reference_optimizer(golden, oracle):
    p0, g1, g2 = golden["sgd/p0"], golden["sgd/g1"], golden["sgd/g2"]
    assert not np.array_equal(golden["sgd/p1"], p0)
    p1, _ = oracle.sgd_step(p0, g1, None, lr=0.01, weight_decay=1e-4)
    np.testing.assert_array_equal(p1, golden["sgd/p1"])
    p2, _ = oracle.sgd_step(p1, g2, None, lr=0.01, weight_decay=1e-4)
    np.testing.assert_array_equal(p2, golden["sgd/p2"])


def test_max_selection_rule_edge_cases(oracle):
    """NaN never wins; a slice with nothing above -inf reports (-inf, 0)
    (strict `>` from -inf: keydnn_reduce_cuda.cu:167-179)."""
    x = np.array([[np.nan, 1.0, 1.0], [-np.inf, -np.inf, -np.inf], [np.nan, np.nan, np.nan]], np.float32)
    val, idx = oracle.max_axis2d(x, 1)
    np.testing.assert_array_equal(val, np.array([1.0, -np.inf, -np.inf], np.float32))
    np.testing.assert_array_equal(idx, np.array([1, 0, 0]))
    xp = np.full((1, 1, 2, 2), np.nan, np.float32)
    y, pidx = oracle.maxpool2d_forward(xp, 2, 2, 0)
    assert np.isneginf(y).all() and pidx.reshape(-1)[0] == 0


# --- activations, unary ops, losses, Adam: the reference's own CPU path ran these ---------------
def test_activations_match_reference_cpu(golden, oracle):
    x, go = golden["act/x"], golden["act/go"]
    cases = {
        "exp": (oracle.exp(x), lambda y: oracle.exp_backward(go, y)),
        "sigmoid": (oracle.sigmoid(x), lambda y: oracle.sigmoid_backward(go, y)),
        "tanh": (oracle.tanh(x), lambda y: oracle.tanh_backward(go, y)),
        "relu": (oracle.relu(x)[0], lambda y: oracle.relu_backward(go, x)),
        "leaky": (oracle.leaky_relu(x, x, 0.1), lambda y: oracle.leaky_relu(go, x, 0.1)),
    }
    for name, (y, bwd) in cases.items():
        np.testing.assert_array_equal(y, golden[f"act/{name}_y"], err_msg=name)
        np.testing.assert_array_equal(bwd(y), golden[f"act/{name}_gx"], err_msg=name)
    for axis, name in ((-1, "softmax1"), (0, "softmax0")):
        y = oracle.softmax(x, axis)
        np.testing.assert_allclose(y, golden[f"act/{name}_y"], rtol=1e-6, atol=1e-8)
        np.testing.assert_allclose(oracle.softmax_backward(go, y, axis), golden[f"act/{name}_gx"], rtol=1e-5, atol=1e-7)
        np.testing.assert_allclose(y.sum(axis), 1.0, rtol=1e-6)


def test_log_sqrt_match_reference_cpu(golden, oracle):
    xp, go = golden["act/xpos"], golden["act/go"]
    np.testing.assert_array_equal(oracle.log(xp), golden["act/log_y"])
    np.testing.assert_array_equal(oracle.log_backward(go, xp), golden["act/log_gx"])
    np.testing.assert_array_equal(oracle.sqrt(xp), golden["act/sqrt_y"])
    np.testing.assert_array_equal(oracle.sqrt_backward(go, oracle.sqrt(xp)), golden["act/sqrt_gx"])


def test_losses_match_reference_cpu(golden, oracle):
    pred, g = golden["loss/pred"], float(golden["loss/g"])
    for name, mean in (("sse", False), ("mse", True)):
        loss, diff = oracle.sqdiff(pred, golden["loss/target"], mean)
        np.testing.assert_allclose(loss, golden[f"loss/{name}_y"], rtol=1e-6)
        gp, gt = oracle.sqdiff_backward(diff, g, mean)
        np.testing.assert_array_equal(gp, golden[f"loss/{name}_gpred"])
        np.testing.assert_array_equal(gt, golden[f"loss/{name}_gtarget"])
    np.testing.assert_allclose(oracle.bce(pred, golden["loss/binary"]), golden["loss/bce_y"], rtol=1e-6)
    np.testing.assert_array_equal(oracle.bce_backward(pred, golden["loss/binary"], g), golden["loss/bce_gpred"])
    np.testing.assert_allclose(oracle.cce(pred, golden["loss/onehot"]), golden["loss/cce_y"], rtol=1e-6)
    np.testing.assert_array_equal(oracle.cce_backward(pred, golden["loss/onehot"], g), golden["loss/cce_gpred"])


@pytest.mark.parametrize("tag,wd", [("adam", 0.0), ("adam_wd", 1e-2)])
def test_adam_matches_reference_cpu_bitwise(golden, oracle, tag, wd):
    p = golden["adam/p0"]
    m, v = np.zeros_like(p), np.zeros_like(p)
    for k in range(3):
        p, m, v = oracle.adam_step(p, golden[f"adam/g{k + 1}"], m, v, k + 1, 1e-2, (0.9, 0.999), 1e-8, wd)
        np.testing.assert_array_equal(p, golden[f"{tag}/p{k + 1}"])
    np.testing.assert_array_equal(m, golden[f"{tag}/m3"])
    np.testing.assert_array_equal(v, golden[f"{tag}/v3"])
