"""exp / log / sqrt, activations, softmax, losses and Adam through the C ABI.

Three checkers: the NumPy oracle (bit-exact wherever no exp / log is involved), the outputs of the
reference's own CPU path (tests/golden), and - the strongest - the reference's own CUDA kernels
compiled unmodified, chained exactly as its Functions chain them: the fused kernels must
reproduce those chains bit for bit."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from _gpu_util import Buf, assert_same_bits, cfloat, native, ref_cuda, suf

pytestmark = pytest.mark.gpu

DTYPES = [np.float32, np.float64]
SIZES = [1, 3, 4, 1023, (1 << 16) + 1, (1 << 20) + 7]
ULP = {np.dtype(np.float32): 2.5e-7, np.dtype(np.float64): 5e-16}


def _x(n, dtype, seed=0, scale=3.0):
    x = (np.random.default_rng(seed).standard_normal(n) * scale).astype(dtype)
    x[: min(n, 4)] = np.array([0.0, -0.0, 1e-3, -1e-3], dtype)[: min(n, 4)]
    return x


def _unary(lib, name, x, *extra):
    dx, dy = Buf(lib, x), Buf(lib, shape=x.shape, dtype=x.dtype, fill=0xFF)
    lib.call(f"keydnn_cuda_{name}_{suf(x.dtype)}", dx.ptr, dy.ptr, *extra, x.size)
    return dy.get()


def _binary(lib, name, a, b, *extra):
    da, db, dy = Buf(lib, a), Buf(lib, b), Buf(lib, shape=a.shape, dtype=a.dtype, fill=0xFF)
    lib.call(f"keydnn_cuda_{name}_{suf(a.dtype)}", da.ptr, db.ptr, dy.ptr, *extra, a.size)
    return dy.get()


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_exp_log_sqrt(oracle, dtype):
    lib = native()
    for n in SIZES:
        x = _x(n, dtype, n)
        np.testing.assert_allclose(_unary(lib, "exp", x), oracle.exp(x), rtol=2 * ULP[np.dtype(dtype)])
        xp = np.abs(x) + dtype(0.01)
        np.testing.assert_allclose(_unary(lib, "log", xp), oracle.log(xp), rtol=2 * ULP[np.dtype(dtype)], atol=1e-7)
        y = _unary(lib, "sqrt", xp)
        assert_same_bits(y, oracle.sqrt(xp))
        g = _x(n, dtype, n + 1, 1.0)
        assert_same_bits(_binary(lib, "sqrt_backward", g, y), oracle.sqrt_backward(g, y))
    special = np.array([np.inf, -np.inf, np.nan, 0.0, -0.0, 88.8, -80.0, 710.0, -700.0], dtype)
    with np.errstate(all="ignore"):
        np.testing.assert_allclose(_unary(lib, "exp", special), np.exp(special), rtol=2 * ULP[np.dtype(dtype)])
        np.testing.assert_allclose(_unary(lib, "log", special), np.log(special), rtol=2 * ULP[np.dtype(dtype)])
        assert_same_bits(_unary(lib, "sqrt", special), np.sqrt(special))


def test_exp_status_codes_follow_the_reference():
    lib = native()
    d = Buf(lib, np.zeros(4, np.float32))
    f = lib.raw("keydnn_cuda_exp_f32")
    assert f(d.ptr, d.ptr, -1) == 1
    assert f(None, None, 0) == 0
    assert f(None, d.ptr, 4) == 2 and f(d.ptr, None, 4) == 2
    assert lib.raw("keydnn_cuda_log_f32")(None, d.ptr, 4) == -1
    assert lib.raw("keydnn_cuda_sigmoid_forward_f64")(d.ptr, d.ptr, -3) == -2


def test_exp_same_bits_as_reference_cuda_kernel():
    ref = ref_cuda()
    if ref is None:
        pytest.skip("reference CUDA library not built")
    lib = native()
    for dtype in DTYPES:
        x = np.concatenate([_x((1 << 20) + 3, dtype, 4, 8.0), np.linspace(-104, 89, 100001).astype(dtype)])
        outs = []
        for L in (lib, ref):
            dx, dy = Buf(L, x), Buf(L, shape=x.shape, dtype=dtype)
            L.call(f"keydnn_cuda_exp_{suf(dtype)}", dx.ptr, dy.ptr, x.size)
            outs.append(dy.get())
        assert_same_bits(outs[0], outs[1])


def _ref_chain_sigmoid(ref, x):
    """SigmoidFn.forward as the reference runs it on CUDA: neg, exp, += 1, fill(1), div."""
    n, s = x.size, suf(x.dtype)
    dx, t, one, y = (Buf(ref, x), Buf(ref, shape=x.shape, dtype=x.dtype), Buf(ref, shape=x.shape, dtype=x.dtype),
                     Buf(ref, shape=x.shape, dtype=x.dtype))
    ref.call(f"keydnn_cuda_neg_{s}", dx.ptr, t.ptr, n)
    ref.call(f"keydnn_cuda_exp_{s}", t.ptr, t.ptr, n)
    ref.call(f"keydnn_cuda_add_scalar_inplace_{s}", t.ptr, cfloat(x.dtype, 1.0), n)
    ref.call(f"keydnn_cuda_fill_{s}", one.ptr, n, cfloat(x.dtype, 1.0))
    ref.call(f"keydnn_cuda_div_{s}", one.ptr, t.ptr, y.ptr, n)
    return y.get()


def _ref_chain_tanh(ref, x):
    """TanhFn.forward: exp(x), neg, exp, sub, add in place, div."""
    n, s = x.size, suf(x.dtype)
    mk = lambda: Buf(ref, shape=x.shape, dtype=x.dtype)   # noqa: E731
    dx, ep, en, num, y = Buf(ref, x), mk(), mk(), mk(), mk()
    ref.call(f"keydnn_cuda_exp_{s}", dx.ptr, ep.ptr, n)
    ref.call(f"keydnn_cuda_neg_{s}", dx.ptr, en.ptr, n)
    ref.call(f"keydnn_cuda_exp_{s}", en.ptr, en.ptr, n)
    ref.call(f"keydnn_cuda_sub_{s}", ep.ptr, en.ptr, num.ptr, n)
    ref.call(f"keydnn_cuda_add_inplace_{s}", ep.ptr, en.ptr, n)
    ref.call(f"keydnn_cuda_div_{s}", num.ptr, ep.ptr, y.ptr, n)
    return y.get()


@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_tanh_same_bits_as_the_reference_kernel_chains(dtype):
    ref = ref_cuda()
    if ref is None:
        pytest.skip("reference CUDA library not built")
    lib = native()
    x = np.concatenate([_x((1 << 18) + 5, dtype, 8, 4.0), np.array([np.inf, -np.inf, np.nan, 90.0, -90.0, 800.0], dtype)])
    assert_same_bits(_unary(lib, "sigmoid_forward", x), _ref_chain_sigmoid(ref, x))
    assert_same_bits(_unary(lib, "tanh_forward", x), _ref_chain_tanh(ref, x))


@pytest.mark.parametrize("dtype", DTYPES)
def test_activations_against_the_oracle(oracle, dtype):
    lib = native()
    tol = dict(rtol=8 * ULP[np.dtype(dtype)], atol=1e-30)
    for n in SIZES:
        x, g = _x(n, dtype, n), _x(n, dtype, n + 7, 1.0)
        y = _unary(lib, "sigmoid_forward", x)
        np.testing.assert_allclose(y, oracle.sigmoid(x), **tol)
        assert_same_bits(_binary(lib, "sigmoid_backward", g, y), oracle.sigmoid_backward(g, y))
        y = _unary(lib, "tanh_forward", x[np.abs(x) < 20] if n > 4 else x)
        xs = x[np.abs(x) < 20] if n > 4 else x
        np.testing.assert_allclose(y, oracle.tanh(xs), rtol=64 * ULP[np.dtype(dtype)], atol=1e-6 if dtype == np.float32 else 1e-14)
        assert_same_bits(_binary(lib, "tanh_backward", g[: y.size], y), oracle.tanh_backward(g[: y.size], y))
        # relu: y and the saved mask; backward from x
        dx, dy, dm = Buf(lib, x), Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF), Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_relu_forward_{suf(dtype)}", dx.ptr, dy.ptr, dm.ptr, n)
        wy, wm = oracle.relu(x)
        assert_same_bits(dy.get(), wy)
        assert_same_bits(dm.get(), wm)
        lib.call(f"keydnn_cuda_relu_forward_{suf(dtype)}", dx.ptr, dy.ptr, None, n)          # mask not wanted
        assert_same_bits(dy.get(), wy)
        assert_same_bits(_binary(lib, "relu_backward", g, x), oracle.relu_backward(g, x))
        assert_same_bits(_unary(lib, "leaky_relu_forward", x, cfloat(dtype, 0.1)), oracle.leaky_relu(x, x, 0.1))
        assert_same_bits(_binary(lib, "leaky_relu_backward", g, x, cfloat(dtype, 0.1)), oracle.leaky_relu(g, x, 0.1))


def test_relu_special_values_follow_x_times_mask(oracle):
    lib = native()
    x = np.array([np.nan, -np.inf, np.inf, -0.0, 0.0, -2.0, 2.0, 1e-45], np.float32)
    with np.errstate(all="ignore"):
        want = oracle.relu(x)[0]                         # -inf * 0 = NaN, -2 * 0 = -0.0: kept, as the reference has it
    dx, dy = Buf(lib, x), Buf(lib, shape=x.shape, dtype=np.float32)
    lib.call("keydnn_cuda_relu_forward_f32", dx.ptr, dy.ptr, None, x.size)
    assert_same_bits(dy.get(), want)


def test_activations_match_reference_cpu_outputs(golden):
    lib = native()
    x, go = golden["act/x"].reshape(-1), golden["act/go"].reshape(-1)
    tol = dict(rtol=2e-6, atol=1e-7)
    y = _unary(lib, "sigmoid_forward", x)
    np.testing.assert_allclose(y, golden["act/sigmoid_y"].reshape(-1), **tol)
    np.testing.assert_allclose(_binary(lib, "sigmoid_backward", go, y), golden["act/sigmoid_gx"].reshape(-1), **tol)
    y = _unary(lib, "tanh_forward", x)
    np.testing.assert_allclose(y, golden["act/tanh_y"].reshape(-1), **tol)
    np.testing.assert_allclose(_binary(lib, "tanh_backward", go, y), golden["act/tanh_gx"].reshape(-1), rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(_unary(lib, "exp", x), golden["act/exp_y"].reshape(-1), **tol)
    assert_same_bits(_binary(lib, "relu_backward", go, x), golden["act/relu_gx"].reshape(-1))
    assert_same_bits(_unary(lib, "leaky_relu_forward", x, ctypes.c_float(0.1)), golden["act/leaky_y"].reshape(-1))
    assert_same_bits(_binary(lib, "leaky_relu_backward", go, x, ctypes.c_float(0.1)), golden["act/leaky_gx"].reshape(-1))
    xp = golden["act/xpos"].reshape(-1)
    np.testing.assert_allclose(_unary(lib, "log", xp), golden["act/log_y"].reshape(-1), **tol)
    y = _unary(lib, "sqrt", xp)
    assert_same_bits(y, golden["act/sqrt_y"].reshape(-1))
    assert_same_bits(_binary(lib, "sqrt_backward", go, y), golden["act/sqrt_gx"].reshape(-1))


def test_unaligned_pointers_take_the_scalar_path(oracle):
    lib = native()
    n = 4099
    x = _x(n + 1, np.float32, 3)
    g = _x(n + 1, np.float32, 4, 1.0)
    dx, dg, dy = Buf(lib, x), Buf(lib, g), Buf(lib, shape=(n + 1,), dtype=np.float32, fill=0)
    lib.call("keydnn_cuda_relu_backward_f32", dg.ptr + 4, dx.ptr + 4, dy.ptr + 4, n)
    assert_same_bits(dy.get()[1:], oracle.relu_backward(g[1:], x[1:]))
    assert dy.get()[0] == 0


# ---------------------------------------------------------------------------------------------
SOFTMAX_SHAPES = [(1, 1, 1), (7, 1, 1), (5, 10, 1), (33, 33, 1), (64, 100, 1), (300, 257, 1), (17, 1000, 1), (9, 1024, 1),
                  (6, 1500, 1), (3, 5000, 1), (2, 60000, 1), (4, 10, 7), (3, 37, 64), (1, 50, 1000), (2000, 2, 1),
                  # rows split over a thread-block cluster (32 KiB and more): 2, 4 and 8 pieces, a ragged last piece,
                  # pieces above 48 KiB, and more rows than resident clusters (every cluster walks several rows)
                  (16, 8192, 1), (8, 16384, 1), (5, 8196, 1), (3, 150000, 1), (4000, 8192, 1),
                  # rows kept in registers (1024 .. 16384 elements in whole packets): every CTA width / packets-per-thread
                  # class, full and ragged last packets
                  (9, 1024, 1), (7, 1028, 1), (6, 2048, 1), (5, 3000, 1), (5, 4096, 1), (7, 4100, 1), (6, 6144, 1),
                  (3, 12000, 1), (2, 16380, 1), (700, 1024, 1)]


@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_forward_backward(oracle, dtype):
    lib = native()
    rtol = 2e-6 if dtype == np.float32 else 1e-13
    for outer, length, inner in SOFTMAX_SHAPES:
        rng = np.random.default_rng(outer * 1000 + length + inner)
        x = (rng.standard_normal((outer, length, inner)) * 4).astype(dtype)
        g = rng.standard_normal(x.shape).astype(dtype)
        dx, dg = Buf(lib, x), Buf(lib, g)
        dy, dgx = Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF), Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_softmax_forward_{suf(dtype)}", dx.ptr, dy.ptr, outer, length, inner)
        y = dy.get()
        want = oracle.softmax(x, 1)          # in the element type: x - max rounds before exp, as in the reference
        np.testing.assert_allclose(y, want, rtol=rtol, atol=1e-30, err_msg=str((outer, length, inner)))
        np.testing.assert_allclose(y.sum(1, dtype=np.float64), 1.0, rtol=1e-5 if dtype == np.float32 else 1e-12)
        lib.call(f"keydnn_cuda_softmax_backward_{suf(dtype)}", dg.ptr, dy.ptr, dgx.ptr, outer, length, inner)
        want_g = oracle.softmax_backward(g.astype(np.float64), y.astype(np.float64), 1)
        np.testing.assert_allclose(dgx.get(), want_g, rtol=rtol * 50, atol=(1e-6 if dtype == np.float32 else 1e-14),
                                   err_msg=str((outer, length, inner)))


def test_softmax_special_rows_and_golden(golden):
    lib = native()
    x = np.zeros((4, 40), np.float32)
    x[0, 3] = np.inf                       # inf - inf = NaN at the maximum itself, 0 elsewhere: the reference's result
    x[1, 5] = np.nan                       # a NaN never wins the max but poisons the sum
    x[2, :] = -np.inf                      # -inf - -inf = NaN everywhere
    x[3, :] = 1000.0                       # large but finite: uniform
    dx, dy = Buf(lib, x), Buf(lib, shape=x.shape, dtype=np.float32)
    lib.call("keydnn_cuda_softmax_forward_f32", dx.ptr, dy.ptr, 4, 40, 1)
    y = dy.get()
    assert np.isnan(y[0, 3]) and np.isnan(y[1]).all() and np.isnan(y[2]).all()
    np.testing.assert_allclose(y[3], 1.0 / 40, rtol=1e-6)
    gx_in, go = golden["act/x"], golden["act/go"]
    for axis, name, view in ((1, "softmax1", (13, 37, 1)), (0, "softmax0", (1, 13, 37))):
        dx, dg = Buf(lib, gx_in), Buf(lib, go)
        dy, dgx = Buf(lib, shape=gx_in.shape, dtype=np.float32), Buf(lib, shape=gx_in.shape, dtype=np.float32)
        lib.call("keydnn_cuda_softmax_forward_f32", dx.ptr, dy.ptr, *view)
        np.testing.assert_allclose(dy.get(), golden[f"act/{name}_y"], rtol=2e-6, atol=1e-9)
        lib.call("keydnn_cuda_softmax_backward_f32", dg.ptr, dy.ptr, dgx.ptr, *view)
        np.testing.assert_allclose(dgx.get(), golden[f"act/{name}_gx"], rtol=1e-4, atol=1e-7)


# ---------------------------------------------------------------------------------------------
def _scalar(lib, dtype):
    return Buf(lib, shape=(1,), dtype=dtype, fill=0xFF)


@pytest.mark.parametrize("dtype", DTYPES)
def test_losses_forward_backward(oracle, dtype):
    lib = native()
    s = suf(dtype)
    rtol = 2e-6 if dtype == np.float32 else 1e-13
    for shape in ((16, 10), (1, 1), (33, 7), (1024, 1000)):
        rng = np.random.default_rng(shape[0] + shape[1])
        n = shape[0] * shape[1]
        pred = rng.uniform(0.05, 0.95, shape).astype(dtype)
        target = rng.standard_normal(shape).astype(dtype)
        binary = (rng.uniform(size=shape) > 0.5).astype(dtype)
        onehot = np.eye(shape[1], dtype=dtype)[rng.integers(0, shape[1], shape[0])]
        gval = dtype(0.7)
        dp, dt, db, do, dgs = Buf(lib, pred), Buf(lib, target), Buf(lib, binary), Buf(lib, onehot), Buf(lib, np.array([gval], dtype))
        for mean in (0, 1):
            ddiff, dl = Buf(lib, shape=shape, dtype=dtype, fill=0xFF), _scalar(lib, dtype)
            lib.call(f"keydnn_cuda_sqdiff_forward_{s}", dp.ptr, dt.ptr, ddiff.ptr, dl.ptr, n, mean)
            wl, wd = oracle.sqdiff(pred, target, bool(mean))
            np.testing.assert_allclose(dl.get()[0], wl, rtol=rtol)
            assert_same_bits(ddiff.get(), wd)
            lib.call(f"keydnn_cuda_sqdiff_forward_{s}", dp.ptr, dt.ptr, None, dl.ptr, n, mean)
            np.testing.assert_allclose(dl.get()[0], wl, rtol=rtol)
            dgp, dgt = Buf(lib, shape=shape, dtype=dtype, fill=0xFF), Buf(lib, shape=shape, dtype=dtype, fill=0xFF)
            scale = (2.0 / n) if mean else 2.0
            for gptr, g in ((dgs.ptr, float(gval)), (None, 1.0)):
                lib.call(f"keydnn_cuda_sqdiff_backward_{s}", ddiff.ptr, gptr, ctypes.c_double(scale), dgp.ptr, dgt.ptr, n)
                wgp, wgt = oracle.sqdiff_backward(wd, g, bool(mean))
                assert_same_bits(dgp.get(), wgp)
                assert_same_bits(dgt.get(), wgt)
        dl, dgp = _scalar(lib, dtype), Buf(lib, shape=shape, dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_bce_forward_{s}", dp.ptr, db.ptr, dl.ptr, n)
        np.testing.assert_allclose(dl.get()[0], oracle.bce(pred, binary), rtol=rtol)
        lib.call(f"keydnn_cuda_bce_backward_{s}", dp.ptr, db.ptr, dgs.ptr, dgp.ptr, n)
        assert_same_bits(dgp.get(), oracle.bce_backward(pred, binary, float(gval)))
        lib.call(f"keydnn_cuda_cce_forward_{s}", dp.ptr, do.ptr, dl.ptr, n, shape[0])
        np.testing.assert_allclose(dl.get()[0], oracle.cce(pred, onehot), rtol=rtol)
        lib.call(f"keydnn_cuda_cce_backward_{s}", dp.ptr, do.ptr, None, dgp.ptr, n, shape[0])
        assert_same_bits(dgp.get(), oracle.cce_backward(pred, onehot, 1.0))


def test_losses_match_reference_cpu_outputs(golden):
    lib = native()
    pred, g = golden["loss/pred"], golden["loss/g"].reshape(1)
    n, batch = pred.size, pred.shape[0]
    dp, dg = Buf(lib, pred), Buf(lib, g)
    dl, dgp, dgt = _scalar(lib, np.float32), Buf(lib, shape=pred.shape, dtype=np.float32), Buf(lib, shape=pred.shape, dtype=np.float32)
    ddiff = Buf(lib, shape=pred.shape, dtype=np.float32)
    dt = Buf(lib, golden["loss/target"])
    for name, mean in (("sse", 0), ("mse", 1)):
        lib.call("keydnn_cuda_sqdiff_forward_f32", dp.ptr, dt.ptr, ddiff.ptr, dl.ptr, n, mean)
        np.testing.assert_allclose(dl.get()[0], golden[f"loss/{name}_y"], rtol=1e-6)
        lib.call("keydnn_cuda_sqdiff_backward_f32", ddiff.ptr, dg.ptr, ctypes.c_double(2.0 / n if mean else 2.0), dgp.ptr, dgt.ptr, n)
        assert_same_bits(dgp.get(), golden[f"loss/{name}_gpred"])
        assert_same_bits(dgt.get(), golden[f"loss/{name}_gtarget"])
    db, do = Buf(lib, golden["loss/binary"]), Buf(lib, golden["loss/onehot"])
    lib.call("keydnn_cuda_bce_forward_f32", dp.ptr, db.ptr, dl.ptr, n)
    np.testing.assert_allclose(dl.get()[0], golden["loss/bce_y"], rtol=1e-6)
    lib.call("keydnn_cuda_bce_backward_f32", dp.ptr, db.ptr, dg.ptr, dgp.ptr, n)
    assert_same_bits(dgp.get(), golden["loss/bce_gpred"])
    lib.call("keydnn_cuda_cce_forward_f32", dp.ptr, do.ptr, dl.ptr, n, batch)
    np.testing.assert_allclose(dl.get()[0], golden["loss/cce_y"], rtol=1e-6)
    lib.call("keydnn_cuda_cce_backward_f32", dp.ptr, do.ptr, dg.ptr, dgp.ptr, n, batch)
    assert_same_bits(dgp.get(), golden["loss/cce_gpred"])


# ---------------------------------------------------------------------------------------------
def _adam_call(lib, dtype, dp, dg, dm, dv, n, step, lr, b1, b2, eps, wd, gscale=1.0):
    c = lambda v: cfloat(dtype, v)   # noqa: E731
    lib.call(f"keydnn_cuda_adam_step_{suf(dtype)}", dp, dg, dm, dv, n, c(lr), c(b1), c(b2), c(eps), c(wd), c(1.0 - b1),
             c(1.0 - b2), c(1.0 - b1 ** step), c(1.0 - b2 ** step), c(gscale))


@pytest.mark.parametrize("dtype", DTYPES)
def test_adam_bit_exact_against_the_oracle(oracle, dtype):
    lib = native()
    for n, wd, off in ((1, 0.0, 0), (53, 1e-2, 0), (4099, 0.0, 1), ((1 << 18) + 3, 1e-4, 0)):
        rng = np.random.default_rng(n)
        p = rng.standard_normal(n + off).astype(dtype)
        m, v = np.zeros_like(p), np.zeros_like(p)
        dp, dm, dv = Buf(lib, p), Buf(lib, m), Buf(lib, v)
        isz = np.dtype(dtype).itemsize
        for step in (1, 2, 3):
            g = (rng.standard_normal(n + off) * 0.1).astype(dtype)
            dg = Buf(lib, g)
            _adam_call(lib, dtype, dp.ptr + off * isz, dg.ptr + off * isz, dm.ptr + off * isz, dv.ptr + off * isz, n, step,
                       1e-2, 0.9, 0.999, 1e-8, wd)
            p[off:], m[off:], v[off:] = oracle.adam_step(p[off:], g[off:], m[off:], v[off:], step, 1e-2, (0.9, 0.999), 1e-8, wd)
            assert_same_bits(dp.get(), p)
            assert_same_bits(dm.get(), m)
            assert_same_bits(dv.get(), v)


@pytest.mark.parametrize("tag,wd", [("adam", 0.0), ("adam_wd", 1e-2)])
def test_adam_matches_reference_cpu_outputs_bitwise(golden, tag, wd):
    lib = native()
    p0 = golden["adam/p0"]
    dp, dm, dv = Buf(lib, p0), Buf(lib, np.zeros_like(p0)), Buf(lib, np.zeros_like(p0))
    for k in range(3):
        dg = Buf(lib, golden[f"adam/g{k + 1}"])
        _adam_call(lib, np.float32, dp.ptr, dg.ptr, dm.ptr, dv.ptr, p0.size, k + 1, 1e-2, 0.9, 0.999, 1e-8, wd)
        assert_same_bits(dp.get(), golden[f"{tag}/p{k + 1}"])
    assert_same_bits(dm.get(), golden[f"{tag}/m3"])
    assert_same_bits(dv.get(), golden[f"{tag}/v3"])


def _ref_chain_softmax(ref, x, g):
    """SoftmaxFn forward / backward exactly as the reference runs them on a CUDA (rows, cols) tensor, axis = 1:
    max -> broadcast_to -> sub -> exp -> sum -> broadcast_to -> div;  mul -> sum -> broadcast_to -> sub -> mul."""
    rows, cols = x.shape
    s, dt = suf(x.dtype), x.dtype
    mk = lambda shape=x.shape: Buf(ref, shape=shape, dtype=dt)   # noqa: E731
    small, full = (ctypes.c_int64 * 2)(rows, 1), (ctypes.c_int64 * 2)(rows, cols)

    keep = []                   # every temporary stays allocated until the results are read back

    def bcast(src):
        dst = mk()
        keep.append(dst)
        ref.call(f"keydnn_cuda_broadcast_to_{s}", src.ptr, dst.ptr, small, 2, full, 2)
        return dst

    dx, dg = Buf(ref, x), Buf(ref, g)
    m, idx = mk((rows,)), Buf(ref, shape=(rows,), dtype=np.int64)
    ref.call(f"keydnn_cuda_max_axis2d_forward_{s}", dx.ptr, m.ptr, idx.ptr, rows, cols, 1)
    shift, e, den, y = mk(), mk(), mk((rows,)), mk()
    ref.call(f"keydnn_cuda_sub_{s}", dx.ptr, bcast(m).ptr, shift.ptr, x.size)
    ref.call(f"keydnn_cuda_exp_{s}", shift.ptr, e.ptr, x.size)
    ref.call(f"keydnn_cuda_sum_axis2d_forward_{s}", e.ptr, den.ptr, rows, cols, 1)
    ref.call(f"keydnn_cuda_div_{s}", e.ptr, bcast(den).ptr, y.ptr, x.size)
    gy, dot, t, gx = mk(), mk((rows,)), mk(), mk()
    ref.call(f"keydnn_cuda_mul_{s}", dg.ptr, y.ptr, gy.ptr, x.size)
    ref.call(f"keydnn_cuda_sum_axis2d_forward_{s}", gy.ptr, dot.ptr, rows, cols, 1)
    ref.call(f"keydnn_cuda_sub_{s}", dg.ptr, bcast(dot).ptr, t.ptr, x.size)
    ref.call(f"keydnn_cuda_mul_{s}", y.ptr, t.ptr, gx.ptr, x.size)
    out = (y.get(), gx.get())
    del keep
    return out


@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_rows_up_to_32_same_bits_as_the_reference_kernel_chain(dtype):
    """Classifier-head rows are reduced in the reference's serial order and divided, not scaled: bit-identical."""
    ref = ref_cuda()
    if ref is None:
        pytest.skip("reference CUDA library not built")
    lib = native()
    for rows, cols in ((1, 1), (5, 2), (300, 3), (256, 10), (1000, 16), (777, 17), (513, 31), (2048, 32)):
        rng = np.random.default_rng(rows + cols)
        x = (rng.standard_normal((rows, cols)) * 3).astype(dtype)
        g = rng.standard_normal((rows, cols)).astype(dtype)
        if rows > 4:
            x[1, 0] = np.nan
            x[2, :] = -np.inf
            x[3, cols - 1] = np.inf
        want_y, want_gx = _ref_chain_softmax(ref, x, g)
        dx, dg = Buf(lib, x), Buf(lib, g)
        dy, dgx = Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF), Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF)
        lib.call(f"keydnn_cuda_softmax_forward_{suf(dtype)}", dx.ptr, dy.ptr, rows, cols, 1)
        lib.call(f"keydnn_cuda_softmax_backward_{suf(dtype)}", dg.ptr, dy.ptr, dgx.ptr, rows, cols, 1)
        assert_same_bits(dy.get(), want_y, err_msg=f"forward {rows}x{cols}")
        assert_same_bits(dgx.get(), want_gx, err_msg=f"backward {rows}x{cols}")
