"""Tensor-level parity: the host mirror's ops and backward closures on the GPU against what the
reference's own Tensor produced on its CPU path for the same inputs (tests/golden/), the level of
the reference's tests/infrastructure/tensors/cuda/test_tensor_*_cuda.py."""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kd():
    import keydnn_v2_b200 as m

    return m


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_arithmetic_autograd_matches_reference(kd, golden, op):
    T = kd.Tensor
    a, b, g = golden["ew/a"], golden["ew/b"], golden["ew/g"]
    ta, tb = T.from_numpy(a, requires_grad=True), T.from_numpy(b, requires_grad=True)
    y = {"add": lambda: ta + tb, "sub": lambda: ta - tb, "mul": lambda: ta * tb, "div": lambda: ta / tb}[op]()
    y.backward(T.from_numpy(g))
    np.testing.assert_array_equal(y.to_numpy(), golden[f"ew/{op}_y"])
    np.testing.assert_allclose(ta.grad.to_numpy(), golden[f"ew/{op}_ga"], rtol=1e-6, atol=0)
    np.testing.assert_allclose(tb.grad.to_numpy(), golden[f"ew/{op}_gb"], rtol=1e-6, atol=0)


def test_neg_compare_scalar_match_reference(kd, golden):
    T = kd.Tensor
    a = golden["ew/a"]
    ta = T.from_numpy(a, requires_grad=True)
    y = -ta
    y.backward(T.from_numpy(golden["ew/g"]))
    np.testing.assert_array_equal(y.to_numpy(), golden["ew/neg_y"])
    np.testing.assert_array_equal(ta.grad.to_numpy(), golden["ew/neg_ga"])
    a2, b2 = T.from_numpy(golden["ew/a2"]), T.from_numpy(golden["ew/b2"])
    for name, fn in (("gt", lambda: a2 > b2), ("ge", lambda: a2 >= b2), ("lt", lambda: a2 < b2), ("le", lambda: a2 <= b2)):
        out = fn()
        assert out.dtype == np.float32 and not out.requires_grad
        np.testing.assert_array_equal(out.to_numpy(), golden[f"ew/{name}_y"])
    t = T.from_numpy(a)
    np.testing.assert_array_equal((t > 0.0).to_numpy(), golden["ew/gt_scalar_y"])
    np.testing.assert_array_equal((t + 1.5).to_numpy(), golden["ew/add_scalar_y"])
    np.testing.assert_array_equal((t * 0.3).to_numpy(), golden["ew/mul_scalar_y"])
    np.testing.assert_array_equal((t / 0.7).to_numpy(), golden["ew/div_scalar_y"])
    np.testing.assert_array_equal((t - 0.25).to_numpy(), golden["ew/sub_scalar_y"])


def test_reductions_autograd_match_reference(kd, golden):
    T = kd.Tensor
    x = golden["red/x"]
    tx = T.from_numpy(x, requires_grad=True)
    y = tx.sum()
    y.backward()
    np.testing.assert_allclose(y.to_numpy(), golden["red/sum_all_y"], rtol=1e-6)
    np.testing.assert_array_equal(tx.grad.to_numpy(), golden["red/sum_all_gx"])
    tx = T.from_numpy(x, requires_grad=True)
    y = tx.mean()
    y.backward()
    np.testing.assert_allclose(y.to_numpy(), golden["red/mean_all_y"], rtol=1e-6)
    np.testing.assert_allclose(tx.grad.to_numpy(), golden["red/mean_all_gx"], rtol=1e-7)
    for axis in (0, 1):
        tx = T.from_numpy(x, requires_grad=True)
        y = tx.sum(axis=axis)
        y.backward(T.from_numpy(golden[f"red/sum_axis{axis}_go"]))
        np.testing.assert_allclose(y.to_numpy(), golden[f"red/sum_axis{axis}_y"], rtol=1e-6, atol=1e-6)
        np.testing.assert_array_equal(tx.grad.to_numpy(), golden[f"red/sum_axis{axis}_gx"])
        tx = T.from_numpy(x, requires_grad=True)
        y = tx.max(axis=axis)
        y.backward(T.from_numpy(golden[f"red/max_axis{axis}_go"]))
        np.testing.assert_array_equal(y.to_numpy(), golden[f"red/max_axis{axis}_y"])
        np.testing.assert_array_equal(tx.grad.to_numpy(), golden[f"red/max_axis{axis}_gx"])


def test_pooling_modules_match_reference(kd, golden):
    from keydnn_v2_b200.pooling import AvgPool2d, GlobalAvgPool2d, MaxPool2d

    T = kd.Tensor
    for name, (k, s, p) in {"k2s2p0": (2, 2, 0), "k3s2p1": (3, 2, 1), "k23s21p10": ((2, 3), (2, 1), (1, 0))}.items():
        x = golden[f"pool/{name}/x"]
        for kind, Mod in (("max", MaxPool2d), ("avg", AvgPool2d)):
            tx = T.from_numpy(x, requires_grad=True)
            y = Mod(k, s, p)(tx)
            y.backward(T.from_numpy(golden[f"pool/{name}/{kind}_go"]))
            np.testing.assert_allclose(y.to_numpy(), golden[f"pool/{name}/{kind}_y"], rtol=1e-6, atol=1e-7)
            np.testing.assert_allclose(tx.grad.to_numpy(), golden[f"pool/{name}/{kind}_gx"], rtol=1e-6, atol=1e-6)
    tx = T.from_numpy(golden["gap/x"], requires_grad=True)
    y = GlobalAvgPool2d()(tx)
    y.backward(T.from_numpy(golden["gap/go"]))
    np.testing.assert_allclose(y.to_numpy(), golden["gap/y"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(tx.grad.to_numpy(), golden["gap/gx"], rtol=1e-6, atol=1e-7)


def test_graph_with_shared_nodes_and_inplace_rules(kd):
    """z = (a*b + a).sum(): a receives two contributions; in-place ops fall back to
    out-of-place + copy for tensors that require grad (arithmetic/_base.py:459-536)."""
    T = kd.Tensor
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((8, 16)), rng.standard_normal((8, 16))
    ta, tb = T.from_numpy(a, requires_grad=True), T.from_numpy(b, requires_grad=True)
    assert ta.dtype == np.float64
    z = (ta * tb + ta).sum()
    z.backward()
    np.testing.assert_allclose(z.item(), (a * b + a).sum(), rtol=1e-12)
    np.testing.assert_allclose(ta.grad.to_numpy(), b + 1.0, rtol=1e-12)
    np.testing.assert_allclose(tb.grad.to_numpy(), a, rtol=1e-12)
    p = T.from_numpy(a, requires_grad=True)
    ptr = p.data
    p -= T.from_numpy(b)
    assert p.data == ptr
    np.testing.assert_array_equal(p.to_numpy(), a - b)
    q = T.from_numpy(a)
    q *= 2.0
    q += T.from_numpy(b)
    np.testing.assert_array_equal(q.to_numpy(), a * 2.0 + b)
    with pytest.raises(ValueError):
        _ = ta + T.from_numpy(rng.standard_normal((4, 4)))
    with pytest.raises(ValueError):
        T.from_numpy(rng.standard_normal((2, 3, 4))).sum(axis=1)


def test_fan_in_of_four_accumulates_without_touching_shared_gradients(kd):
    """u = a + a + a + a: four contributions meet at `a`, all the very same upstream tensor (add's backward
    returns grad_out itself).  The third and fourth are added in place into a private sum; the shared upstream
    gradient must come out unchanged."""
    T = kd.Tensor
    rng = np.random.default_rng(3)
    a = rng.standard_normal((5, 7)).astype(np.float32)
    g = rng.standard_normal((5, 7)).astype(np.float32)
    ta = T.from_numpy(a, requires_grad=True)
    tg = T.from_numpy(g)
    u = ta + ta + ta + ta
    u.backward(tg)
    np.testing.assert_array_equal(tg.to_numpy(), g)
    np.testing.assert_array_equal(ta.grad.to_numpy(), ((g + g) + g) + g)
    # a second backward on a fresh graph adds to .grad out of place: the old .grad object keeps its values
    old = ta.grad
    (ta * 2.0).backward(tg)
    np.testing.assert_array_equal(old.to_numpy(), ((g + g) + g) + g)
    np.testing.assert_array_equal(ta.grad.to_numpy(), (((g + g) + g) + g) + g * np.float32(2.0))


def test_allocator_reuses_blocks(kd):
    import ctypes

    lib = kd.load()
    st = (ctypes.c_uint64 * 4)()
    t = kd.Tensor.zeros((1 << 20,))
    del t
    lib.call("keydnn_cuda_pool_stats", st)
    before = st[2]
    for _ in range(50):
        t = kd.Tensor.zeros((1 << 20,))
        del t
    lib.call("keydnn_cuda_pool_stats", st)
    assert st[2] == before, "temporaries of one size must come from the pool, not from cudaMalloc"
