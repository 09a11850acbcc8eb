"""Parity at the full benchmark sizes.  The oracle is fast enough to check most of them directly;
on top of that, size-independent properties: every max equals the input at its recorded position,
gradients conserve the upstream mass, average-pool backward is the adjoint of forward, reductions
are linear, and a sharded (two half-matrices) evaluation agrees with the whole."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from _gpu_util import Buf, assert_same_bits, native

pytestmark = pytest.mark.gpu


def test_config0_maxpool_32x64x112x112(oracle):
    lib = native()
    N, C, H, W = 32, 64, 112, 112
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    go = rng.standard_normal((N, C, H // 2, W // 2)).astype(np.float32)
    dx, dgo = Buf(lib, x), Buf(lib, go)
    dy, di = Buf(lib, shape=go.shape, dtype=np.float32), Buf(lib, shape=go.shape, dtype=np.int64)
    dgx = Buf(lib, shape=x.shape, dtype=np.float32, fill=0xFF)
    lib.call("keydnn_cuda_maxpool2d_forward_ex_f32", dx.ptr, dy.ptr, di.ptr, N, C, H, W, H // 2, W // 2, 2, 2, 2, 2, 0, 0)
    lib.call("keydnn_cuda_maxpool2d_backward_ex_f32", dgo.ptr, di.ptr, dgx.ptr, N, C, H, W, H // 2, W // 2, 2, 2, 2, 2, 0, 0)
    y, idx, gx = dy.get(), di.get(), dgx.get()
    y_w, idx_w = oracle.maxpool2d_forward(x, 2, 2, 0)
    np.testing.assert_array_equal(y, y_w)
    np.testing.assert_array_equal(idx, idx_w)
    assert_same_bits(gx, oracle.maxpool2d_backward(go, idx_w, x.shape, 0))
    # properties: the value at the recorded position is the maximum; the gradient keeps every go exactly once
    flat = x.reshape(N * C, H * W)
    np.testing.assert_array_equal(np.take_along_axis(flat, idx.reshape(N * C, -1), 1).reshape(y.shape), y)
    assert np.count_nonzero(gx) == np.count_nonzero(go)
    np.testing.assert_allclose(gx.sum(dtype=np.float64), go.sum(dtype=np.float64), rtol=1e-9)


@pytest.mark.parametrize("dtype,shape", [(np.float32, (8192, 8192)), (np.float64, (4096, 4096))])
def test_config1_reductions_full_size(oracle, dtype, shape):
    lib = native()
    s = "f32" if dtype == np.float32 else "f64"
    rows, cols = shape
    rng = np.random.default_rng(1)
    x = rng.standard_normal(shape).astype(dtype)
    x64 = x.astype(np.float64)
    dx = Buf(lib, x)
    tol = dict(rtol=1e-5, atol=1e-4) if dtype == np.float32 else dict(rtol=1e-12, atol=1e-10)
    halves = []
    for axis in (0, 1):
        n_out = cols if axis == 0 else rows
        dy, di = Buf(lib, shape=(n_out,), dtype=dtype), Buf(lib, shape=(n_out,), dtype=np.int64)
        lib.call(f"keydnn_cuda_sum_axis2d_forward_{s}", dx.ptr, dy.ptr, rows, cols, axis)
        np.testing.assert_allclose(dy.get(), x64.sum(axis), **tol)
        lib.call(f"keydnn_cuda_mean_axis2d_forward_{s}", dx.ptr, dy.ptr, rows, cols, axis)
        np.testing.assert_allclose(dy.get(), x64.mean(axis), **tol)
        lib.call(f"keydnn_cuda_max_axis2d_forward_{s}", dx.ptr, dy.ptr, di.ptr, rows, cols, axis)
        np.testing.assert_array_equal(dy.get(), x.max(axis))
        np.testing.assert_array_equal(di.get(), x.argmax(axis))
        dgo = Buf(lib, np.ones(n_out, dtype))
        dgx = Buf(lib, shape=shape, dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_max_axis2d_backward_ex_{s}", dgo.ptr, di.ptr, dgx.ptr, rows, cols, axis)
        gx = dgx.get()
        assert gx.sum() == n_out and np.count_nonzero(gx) == n_out              # one 1 per reduced slice
        np.testing.assert_array_equal(gx.argmax(axis), x.argmax(axis))
        lib.call(f"keydnn_cuda_sum_axis2d_backward_{s}", dgo.ptr, dgx.ptr, rows, cols, axis)
        assert (dgx.get() == 1).all()
    dy1, di1 = Buf(lib, shape=(1,), dtype=dtype), Buf(lib, shape=(1,), dtype=np.int64)
    lib.call(f"keydnn_cuda_sum_all_{s}", dx.ptr, dy1.ptr, rows * cols)
    total = dy1.get()[0]
    np.testing.assert_allclose(total, x64.sum(), **tol)
    lib.call(f"keydnn_cuda_mean_all_{s}", dx.ptr, dy1.ptr, rows * cols)
    np.testing.assert_allclose(dy1.get()[0], x64.mean(), rtol=tol["rtol"], atol=1e-9)
    lib.call(f"keydnn_cuda_max_all_forward_{s}", dx.ptr, dy1.ptr, di1.ptr, rows * cols)
    assert dy1.get()[0] == x.max() and di1.get()[0] == x.argmax()
    # sharding property: the two half-matrices sum to the whole (what the multi-GPU exchange relies on)
    half = rows // 2 * cols
    isz = np.dtype(dtype).itemsize
    for off in (0, half):
        lib.call(f"keydnn_cuda_sum_all_{s}", dx.ptr + off * isz, dy1.ptr, half)
        halves.append(float(dy1.get()[0]))
    np.testing.assert_allclose(halves[0] + halves[1], float(total), **tol)
    # linearity: sum(-x) == -sum(x) bit for bit (the kernel adds in a fixed order)
    dneg = Buf(lib, shape=shape, dtype=dtype)
    lib.call(f"keydnn_cuda_neg_{s}", dx.ptr, dneg.ptr, rows * cols)
    lib.call(f"keydnn_cuda_sum_all_{s}", dneg.ptr, dy1.ptr, rows * cols)
    assert dy1.get()[0] == -total


def test_config2_elementwise_2pow28_and_sgd(oracle):
    lib = native()
    n = 1 << 28
    rng = np.random.default_rng(2)
    a = rng.standard_normal(n, dtype=np.float32)
    b = rng.uniform(0.5, 2.0, n).astype(np.float32)
    da, db, dy = Buf(lib, a), Buf(lib, b), Buf(lib, shape=(n,), dtype=np.float32)
    for op in ("add", "sub", "mul", "div", "gt"):
        lib.call(f"keydnn_cuda_{op}_f32", da.ptr, db.ptr, dy.ptr, n)
        assert_same_bits(dy.get(), oracle.binary(op, a, b), err_msg=op)
    lib.call("keydnn_cuda_neg_f32", da.ptr, dy.ptr, n)
    assert_same_bits(dy.get(), oracle.neg(a))
    dga, dgb = Buf(lib, shape=(n,), dtype=np.float32), Buf(lib, shape=(n,), dtype=np.float32)
    lib.call("keydnn_cuda_div_backward_f32", dy.ptr, da.ptr, db.ptr, dga.ptr, dgb.ptr, n)
    g = oracle.neg(a)
    want = oracle.div_backward(g, a, b)
    assert_same_bits(dga.get(), want[0])
    assert_same_bits(dgb.get(), want[1])
    del da, db, dy, dga, dgb
    n = 25_165_824
    p = rng.standard_normal(n, dtype=np.float32)
    g = (rng.standard_normal(n, dtype=np.float32) * np.float32(1e-2))
    v = np.zeros(n, np.float32)
    dp, dg, dv = Buf(lib, p), Buf(lib, g), Buf(lib, v)
    for _ in range(2):
        lib.call("keydnn_cuda_sgd_momentum_step_f32", dp.ptr, dg.ptr, dv.ptr, n, ctypes.c_float(0.01), ctypes.c_float(0.9),
                 ctypes.c_float(1e-4), ctypes.c_float(1.0))
        p, v = oracle.sgd_step(p, g, v, 0.01, 0.9, 1e-4)
    assert_same_bits(dp.get(), p)
    assert_same_bits(dv.get(), v)


def test_config3_avgpool_256x256x56x56_and_global_avgpool(oracle):
    lib = native()
    N, C, H, W = 256, 256, 56, 56
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    go = rng.standard_normal((N, C, 28, 28)).astype(np.float32)
    dx, dgo = Buf(lib, x), Buf(lib, go)
    dy, dgx = Buf(lib, shape=go.shape, dtype=np.float32), Buf(lib, shape=x.shape, dtype=np.float32, fill=0xFF)
    lib.call("keydnn_cuda_avgpool2d_forward_ex_f32", dx.ptr, dy.ptr, N, C, H, W, 28, 28, 3, 3, 2, 2, 1, 1)
    lib.call("keydnn_cuda_avgpool2d_backward_ex_f32", dgo.ptr, dgx.ptr, N, C, H, W, 28, 28, 3, 3, 2, 2, 1, 1)
    y, gx = dy.get(), dgx.get()
    sl = slice(0, 16)                                           # direct oracle check on 16 images (the rest by properties)
    assert_same_bits(y[sl], oracle.avgpool2d_forward(x[sl], 3, 2, 1))
    assert_same_bits(gx[sl], oracle.avgpool2d_backward(go[sl], x[sl].shape, 3, 2, 1))
    assert_same_bits(y[-4:], oracle.avgpool2d_forward(x[-4:], 3, 2, 1))
    assert_same_bits(gx[-4:], oracle.avgpool2d_backward(go[-4:], x[-4:].shape, 3, 2, 1))
    # adjoint identity <avg(x), go> == <x, avg^T(go)> over the whole tensor
    lhs = np.einsum("nchw,nchw->", y.astype(np.float64), go.astype(np.float64))
    rhs = np.einsum("nchw,nchw->", x.astype(np.float64), gx.astype(np.float64))
    np.testing.assert_allclose(lhs, rhs, rtol=1e-6)
    del dx, dgo, dy, dgx
    N, C, H, W = 256, 2048, 7, 7
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    go = rng.standard_normal((N, C, 1, 1)).astype(np.float32)
    dx, dgo = Buf(lib, x), Buf(lib, go)
    dy, dgx = Buf(lib, shape=go.shape, dtype=np.float32), Buf(lib, shape=x.shape, dtype=np.float32, fill=0xFF)
    lib.call("keydnn_cuda_global_avgpool2d_forward_f32", dx.ptr, dy.ptr, N, C, H, W)
    lib.call("keydnn_cuda_global_avgpool2d_backward_f32", dgo.ptr, dgx.ptr, N, C, H, W)
    assert_same_bits(dy.get(), oracle.global_avgpool2d_forward(x))
    assert_same_bits(dgx.get(), oracle.global_avgpool2d_backward(go, x.shape))
