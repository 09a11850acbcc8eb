"""Reductions and their gradients through the C ABI.

Bars: max values, int64 first-occurrence indices and every gradient kernel bit-exact; sums and
means within the reference's own tolerances (tests/infrastructure/ops/_cuda_test_utils.py:106-136:
f32 rtol 1e-5 / atol 1e-6, f64 1e-12; large f32 sums rtol 2e-5 / atol 1e-4,
native_cuda/test_reduce_ctypes.py:216-221) of the float64 oracle.
"""
from __future__ import annotations

import numpy as np
import pytest

from _gpu_util import Buf, assert_same_bits, native, ref_cuda, suf

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (1, 7), (7, 1), (5, 12), (33, 129), (257, 64), (64, 2048), (300, 4100), (1000, 31), (2050, 520)]


def _sum_tol(dtype, n):
    if np.dtype(dtype) == np.float64:
        return dict(rtol=1e-12, atol=1e-10)
    return dict(rtol=2e-5, atol=1e-4) if n >= 100_000 else dict(rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_sum_mean_all_and_fill_backward(oracle, dtype):
    lib = native()
    s = suf(dtype)
    rng = np.random.default_rng(0)
    for n in (1, 3, 1000, 4097, (1 << 20) + 5, 5_000_003):
        x = rng.standard_normal(n).astype(dtype)
        dx, dy = Buf(lib, x), Buf(lib, shape=(1,), dtype=dtype)
        lib.call(f"keydnn_cuda_sum_all_{s}", dx.ptr, dy.ptr, n)
        first = dy.get()
        np.testing.assert_allclose(first[0], oracle.sum_all(x), **_sum_tol(dtype, n))
        lib.call(f"keydnn_cuda_sum_all_{s}", dx.ptr, dy.ptr, n)
        assert_same_bits(dy.get(), first)            # deterministic, and the ticket counter reset
        lib.call(f"keydnn_cuda_mean_all_{s}", dx.ptr, dy.ptr, n)
        np.testing.assert_allclose(dy.get()[0], oracle.mean_all(x), rtol=_sum_tol(dtype, n)["rtol"],
                                   atol=_sum_tol(dtype, n)["atol"] / n)
        go = np.array([1.7], dtype)
        dgo, dgx = Buf(lib, go), Buf(lib, shape=(n,), dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_sum_backward_fill_{s}", dgo.ptr, dgx.ptr, n)
        assert_same_bits(dgx.get(), oracle.sum_backward_fill(go, n))
        lib.call(f"keydnn_cuda_mean_backward_fill_{s}", dgo.ptr, dgx.ptr, n)
        assert_same_bits(dgx.get(), oracle.mean_backward_fill(go, n))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape", SHAPES)
def test_sum_mean_axis2d(oracle, shape, dtype):
    lib = native()
    s = suf(dtype)
    rows, cols = shape
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal(shape).astype(dtype)
    dx = Buf(lib, x)
    for axis in (0, 1):
        n_out = cols if axis == 0 else rows
        dy = Buf(lib, shape=(n_out,), dtype=dtype)
        lib.call(f"keydnn_cuda_sum_axis2d_forward_{s}", dx.ptr, dy.ptr, rows, cols, axis)
        np.testing.assert_allclose(dy.get(), oracle.sum_axis2d(x, axis), **_sum_tol(dtype, 1))
        lib.call(f"keydnn_cuda_mean_axis2d_forward_{s}", dx.ptr, dy.ptr, rows, cols, axis)
        np.testing.assert_allclose(dy.get(), oracle.mean_axis2d(x, axis), **_sum_tol(dtype, 1))
        go = rng.standard_normal(n_out).astype(dtype)
        dgo, dgx = Buf(lib, go), Buf(lib, shape=shape, dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_sum_axis2d_backward_{s}", dgo.ptr, dgx.ptr, rows, cols, axis)
        assert_same_bits(dgx.get(), oracle.sum_axis2d_backward(go, rows, cols, axis))
        lib.call(f"keydnn_cuda_mean_axis2d_backward_{s}", dgo.ptr, dgx.ptr, rows, cols, axis)
        assert_same_bits(dgx.get(), oracle.mean_axis2d_backward(go, rows, cols, axis))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape", SHAPES)
def test_max_axis2d_forward_backward_bit_exact(oracle, shape, dtype):
    lib = native()
    s = suf(dtype)
    rows, cols = shape
    rng = np.random.default_rng(rows * 3 + cols)
    for quant in (None, 2):                      # quantised -> many ties: first index must win
        x = rng.standard_normal(shape).astype(dtype)
        if quant:
            x = (np.round(x * quant) / quant).astype(dtype)
        dx = Buf(lib, x)
        for axis in (0, 1):
            n_out = cols if axis == 0 else rows
            dy, di = Buf(lib, shape=(n_out,), dtype=dtype), Buf(lib, shape=(n_out,), dtype=np.int64)
            lib.call(f"keydnn_cuda_max_axis2d_forward_{s}", dx.ptr, dy.ptr, di.ptr, rows, cols, axis)
            val, idx = oracle.max_axis2d(x, axis)
            np.testing.assert_array_equal(dy.get(), val)
            np.testing.assert_array_equal(di.get(), idx)
            go = rng.standard_normal(n_out).astype(dtype)
            want = oracle.max_axis2d_backward(go, idx, rows, cols, axis)
            dgo = Buf(lib, go)
            dgx = Buf(lib, shape=shape, dtype=dtype, fill=0xFF)
            lib.call(f"keydnn_cuda_max_axis2d_backward_ex_{s}", dgo.ptr, di.ptr, dgx.ptr, rows, cols, axis)
            assert_same_bits(dgx.get(), want)
            dgz = Buf(lib, shape=shape, dtype=dtype, fill=0)     # reference entry: caller zero-fills
            lib.call(f"keydnn_cuda_max_axis2d_backward_{s}", dgo.ptr, di.ptr, dgz.ptr, rows, cols, axis)
            assert_same_bits(dgz.get(), want)


@pytest.mark.parametrize("shape", [(1000, 2500), (4096, 4096), (513, 3072), (2047, 4104)])
def test_fp64_column_reductions_through_the_cluster_kernels(oracle, shape):
    """Shapes for which the row chunks of a column stripe form one thread-block cluster (8-byte elements, about
    sixteen chunks per stripe fill the machine) and the fold goes through distributed shared memory: ragged last
    stripe, ragged last chunk, ties, NaN and -inf columns; sums to rounding, maxima and first rows exactly, twice
    in a row with the same bits."""
    lib = native()
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal(shape)
    x[:, 3] = -np.inf
    x[:, 5] = np.nan
    x[::7, 11] = 4.25                                 # ties: the first of them must win
    x[rows // 2, 17] = np.nan
    x[rows - 1, cols - 1] = 99.0                      # last row of the last (ragged) chunk and stripe
    dx = Buf(lib, x)
    dy, di = Buf(lib, shape=(cols,), dtype=np.float64, fill=0xFF), Buf(lib, shape=(cols,), dtype=np.int64, fill=0xFF)
    clean = np.where(np.isnan(x), 0.0, x)
    clean[:, 3] = 0.0
    dc = Buf(lib, clean)
    for _ in range(2):
        lib.call("keydnn_cuda_max_axis2d_forward_f64", dx.ptr, dy.ptr, di.ptr, rows, cols, 0)
        val, idx = oracle.max_axis2d(x, 0)
        np.testing.assert_array_equal(dy.get(), val)
        np.testing.assert_array_equal(di.get(), idx)
    assert di.get()[11] == 0 and di.get()[cols - 1] == rows - 1 and di.get()[3] == 0 and dy.get()[5] == -np.inf
    first = None
    for _ in range(2):
        lib.call("keydnn_cuda_sum_axis2d_forward_f64", dc.ptr, dy.ptr, rows, cols, 0)
        got = dy.get()
        np.testing.assert_allclose(got, oracle.sum_axis2d(clean, 0), rtol=1e-12, atol=1e-10)
        if first is not None:
            assert_same_bits(got, first)
        first = got
    lib.call("keydnn_cuda_mean_axis2d_forward_f64", dc.ptr, dy.ptr, rows, cols, 0)
    np.testing.assert_allclose(dy.get(), oracle.mean_axis2d(clean, 0), rtol=1e-12, atol=1e-12)
    lib.call("keydnn_cuda_sum_axis2d_forward_f64", dx.ptr, dy.ptr, rows, cols, 0)      # NaN / -inf propagate as in NumPy
    got = dy.get()
    assert np.isnan(got[5]) and got[3] == -np.inf and np.isnan(got[17])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_full_reductions_over_many_tiles(oracle, dtype):
    """Sizes around the tile kernels' limits: one tile, a ragged last tile, more tiles than one fold round takes
    (4096), more than two rounds' worth (the tiles then grow), with 1-3 trailing elements; the maximum sits in the
    last tile / the tail and is tied with an earlier element."""
    lib = native()
    s = suf(dtype)
    rng = np.random.default_rng(77)
    for n in (8192, 8192 * 3 + 1029, 8192 * 4096 + 3, 8192 * 4100 + 2, 8192 * 9000 + 1):
        x = rng.standard_normal(n).astype(dtype)
        x[n - 1] = x[n // 3] = 7.5
        dx, dy, di = Buf(lib, x), Buf(lib, shape=(1,), dtype=dtype), Buf(lib, shape=(1,), dtype=np.int64)
        lib.call(f"keydnn_cuda_sum_all_{s}", dx.ptr, dy.ptr, n)
        np.testing.assert_allclose(dy.get()[0], np.sum(x.astype(np.float64)), **_sum_tol(dtype, n))
        lib.call(f"keydnn_cuda_max_all_forward_{s}", dx.ptr, dy.ptr, di.ptr, n)
        assert dy.get()[0] == 7.5 and di.get()[0] == n // 3
        x[n // 3] = 0.0
        dx2 = Buf(lib, x)
        lib.call(f"keydnn_cuda_max_all_forward_{s}", dx2.ptr, dy.ptr, di.ptr, n)
        assert dy.get()[0] == 7.5 and di.get()[0] == n - 1
        del dx, dx2


def test_max_nan_inf_rules(oracle):
    lib = native()
    x = np.array([[np.nan, 1.0, 1.0, -2.0], [-np.inf] * 4, [np.nan] * 4, [np.inf, 5.0, np.inf, 0.0]], np.float32)
    dx = Buf(lib, x)
    for axis in (0, 1):
        n_out = 4
        dy, di = Buf(lib, shape=(n_out,), dtype=np.float32), Buf(lib, shape=(n_out,), dtype=np.int64)
        lib.call("keydnn_cuda_max_axis2d_forward_f32", dx.ptr, dy.ptr, di.ptr, 4, 4, axis)
        val, idx = oracle.max_axis2d(x, axis)
        np.testing.assert_array_equal(dy.get(), val)
        np.testing.assert_array_equal(di.get(), idx)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_max_all(oracle, dtype):
    lib = native()
    s = suf(dtype)
    rng = np.random.default_rng(4)
    for n in (1, 5, 4099, (1 << 20) + 1):
        x = (np.round(rng.standard_normal(n) * 4) / 4).astype(dtype)
        dx, dy, di = Buf(lib, x), Buf(lib, shape=(1,), dtype=dtype), Buf(lib, shape=(1,), dtype=np.int64)
        lib.call(f"keydnn_cuda_max_all_forward_{s}", dx.ptr, dy.ptr, di.ptr, n)
        val, idx = oracle.max_all(x)
        assert dy.get()[0] == val and di.get()[0] == idx
        go = np.array([0.5], dtype)
        dgo, dgx = Buf(lib, go), Buf(lib, shape=(n,), dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_max_all_backward_{s}", dgo.ptr, di.ptr, dgx.ptr, n)
        assert_same_bits(dgx.get(), oracle.max_all_backward(go, idx, n))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", [
    ((6, 5, 4, 3), (1, 5, 1, 1)), ((16, 8, 32, 32), (1, 8, 1, 1)), ((4, 6), (1, 6)), ((4, 6), (4, 1)),
    ((3, 4, 5), (3, 1, 5)), ((2, 3, 4), (2, 3, 4)), ((7, 9), (1, 1)), ((2, 3, 4, 5), (2, 1, 4, 1)),
])
def test_sum_to_shape_and_broadcast_to(oracle, case, dtype):
    lib = native()
    s = suf(dtype)
    in_shape, out_shape = case
    rng = np.random.default_rng(len(in_shape))
    x = rng.standard_normal(in_shape).astype(dtype)
    ins, outs = np.asarray(in_shape, np.int64), np.asarray(out_shape, np.int64)
    dx, dy = Buf(lib, x), Buf(lib, shape=out_shape, dtype=dtype)
    for _ in range(2):                                # twice: ticket counters must come back to zero
        lib.call(f"keydnn_cuda_sum_to_shape_{s}", dx.ptr, dy.ptr, ins.ctypes.data, outs.ctypes.data, len(in_shape))
        np.testing.assert_allclose(dy.get(), oracle.sum_to_shape(x, out_shape), **_sum_tol(dtype, 1))
    small = rng.standard_normal(out_shape).astype(dtype)
    ds, db = Buf(lib, small), Buf(lib, shape=in_shape, dtype=dtype, fill=0xFF)
    lib.call(f"keydnn_cuda_broadcast_to_{s}", ds.ptr, db.ptr, outs.ctypes.data, len(out_shape), ins.ctypes.data,
             len(in_shape))
    assert_same_bits(db.get(), oracle.broadcast_to(small, in_shape))


def test_bias_add_and_transpose(oracle):
    lib = native()
    rng = np.random.default_rng(8)
    x, b = rng.standard_normal((37, 10)).astype(np.float32), rng.standard_normal(10).astype(np.float32)
    dx, db, dy = Buf(lib, x), Buf(lib, b), Buf(lib, shape=x.shape, dtype=np.float32)
    lib.call("keydnn_cuda_bias_add_f32", dx.ptr, db.ptr, dy.ptr, 37, 10)
    assert_same_bits(dy.get(), oracle.bias_add(x, b))
    lib.call("keydnn_cuda_bias_add_inplace_f32", dx.ptr, db.ptr, 37, 10)
    assert_same_bits(dx.get(), oracle.bias_add(x, b))
    for shape in ((64, 10), (33, 70), (1, 5)):
        m = rng.standard_normal(shape).astype(np.float64)
        dm, dt = Buf(lib, m), Buf(lib, shape=shape[::-1], dtype=np.float64)
        lib.call("keydnn_cuda_transpose2d_f64", dm.ptr, dt.ptr, shape[0], shape[1])
        np.testing.assert_array_equal(dt.get(), m.T)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_bias_add_and_transpose_packet_paths(oracle, dtype):
    """Shapes that take the 4-element packet kernels (extents multiples of 4) next to ragged ones."""
    lib = native()
    s = "f32" if dtype == np.float32 else "f64"
    rng = np.random.default_rng(18)
    for batch, out in ((1, 4), (5, 8), (257, 12), (300, 1000), (4096, 64), (3, 4096), (7, 6)):
        x, b = rng.standard_normal((batch, out)).astype(dtype), rng.standard_normal(out).astype(dtype)
        dx, db, dy = Buf(lib, x), Buf(lib, b), Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_bias_add_{s}", dx.ptr, db.ptr, dy.ptr, batch, out)
        assert_same_bits(dy.get(), oracle.bias_add(x, b))
        lib.call(f"keydnn_cuda_bias_add_inplace_{s}", dx.ptr, db.ptr, batch, out)
        assert_same_bits(dx.get(), oracle.bias_add(x, b))
    for shape in ((4, 4), (64, 64), (128, 60), (60, 128), (68, 132), (1000, 36), (512, 2048), (4, 1000), (64, 66)):
        m = rng.standard_normal(shape).astype(dtype)
        dm, dt = Buf(lib, m), Buf(lib, shape=shape[::-1], dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_transpose2d_{s}", dm.ptr, dt.ptr, shape[0], shape[1])
        np.testing.assert_array_equal(dt.get(), m.T, err_msg=str(shape))


def test_guards_follow_the_reference():
    lib = native()
    d = Buf(lib, np.zeros(16, np.float32))
    assert lib.raw("keydnn_cuda_sum_all_f32")(None, d.ptr, 4) == -1
    assert lib.raw("keydnn_cuda_sum_all_f32")(d.ptr, d.ptr, 0) == -2
    assert lib.raw("keydnn_cuda_sum_axis2d_forward_f32")(d.ptr, d.ptr, 4, 4, 2) == -3
    assert lib.raw("keydnn_cuda_max_axis2d_forward_f32")(d.ptr, d.ptr, None, 4, 4, 0) == -1
    assert lib.raw("keydnn_cuda_maxpool2d_forward_f32")(None, d.ptr, d.ptr, 1, 1, 4, 4, 2, 2, 2, 2, 2, 2) == -1
    assert lib.raw("keydnn_cuda_maxpool2d_forward_f32")(d.ptr, d.ptr, d.ptr, 0, 1, 4, 4, 2, 2, 2, 2, 2, 2) == -2
    assert lib.raw("keydnn_cuda_maxpool2d_forward_f32")(d.ptr, d.ptr, d.ptr, 1, 1, 4, 4, 2, 2, 2, 2, 0, 2) == -4


def test_same_results_as_reference_cuda_kernels(oracle):
    ref = ref_cuda()
    if ref is None:
        pytest.skip("reference CUDA library not built")
    lib = native()
    rows, cols = 300, 520
    rng = np.random.default_rng(17)
    x = (np.round(rng.standard_normal((rows, cols)) * 4) / 4).astype(np.float32)
    res = []
    for L in (lib, ref):
        dx = Buf(L, x)
        out = []
        for axis in (0, 1):
            n_out = cols if axis == 0 else rows
            dy, di = Buf(L, shape=(n_out,), dtype=np.float32), Buf(L, shape=(n_out,), dtype=np.int64)
            L.call("keydnn_cuda_max_axis2d_forward_f32", dx.ptr, dy.ptr, di.ptr, rows, cols, axis)
            ds = Buf(L, shape=(n_out,), dtype=np.float32)
            L.call("keydnn_cuda_sum_axis2d_forward_f32", dx.ptr, ds.ptr, rows, cols, axis)
            out += [dy.get(), di.get(), ds.get()]
        dsum = Buf(L, shape=(1,), dtype=np.float32)
        L.call("keydnn_cuda_sum_all_f32", dx.ptr, dsum.ptr, rows * cols)
        out.append(dsum.get())
        res.append(out)
    for k in (0, 1, 3, 4):
        np.testing.assert_array_equal(res[0][k], res[1][k])
    for k in (2, 5, 6):
        np.testing.assert_allclose(res[0][k], res[1][k], rtol=2e-5, atol=1e-3)
