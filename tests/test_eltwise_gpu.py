"""Elementwise family through the C ABI against the CPU oracle and the reference CUDA kernels.

Bars (bit-level): add/sub/mul/div, neg, compares, scalar and in-place variants, fill and the
fused SGD step are all bit-identical to the oracle (one IEEE op per element).
Sizes exercise the 16-byte packet path, its ragged tail and the unaligned fallback, as the
reference's own ctypes tests do (tests/infrastructure/native_cuda/ops/test_tensor_arithmetic_ctypes.py).
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from _gpu_util import Buf, assert_same_bits, cfloat, native, ref_cuda, suf

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 4, 5, 1023, 1024, 1025, 4096 + 7, (1 << 20) + 3]
BINARY = ["add", "sub", "mul", "div", "gt", "ge", "lt", "le", "eq", "ne"]


def _inputs(n, dtype, seed=0):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal(n).astype(dtype)
    b = rng.uniform(0.5, 2.0, n).astype(dtype)
    if n >= 8:  # specials and ties
        a[1], a[2], a[3], a[5] = np.nan, np.inf, -0.0, b[5]
        b[2] = np.inf
    return a, b


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("op", BINARY)
def test_binary_bit_exact(oracle, op, dtype):
    lib = native()
    for n in SIZES:
        a, b = _inputs(n, dtype, n)
        want = oracle.binary(op, a, b)
        da, db = Buf(lib, a), Buf(lib, b)
        dy = Buf(lib, shape=(n,), dtype=want.dtype)
        lib.call(f"keydnn_cuda_{op}_{suf(dtype)}", da.ptr, db.ptr, dy.ptr, n)
        got = dy.get()
        assert got.dtype == want.dtype
        assert_same_bits(got, want, err_msg=f"{op} n={n}")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_unaligned_pointers_take_scalar_path(oracle, dtype):
    lib = native()
    n = 1000
    a, b = _inputs(n + 1, dtype, 7)
    da, db, dy = Buf(lib, a), Buf(lib, b), Buf(lib, shape=(n + 1,), dtype=dtype, fill=0)
    isz = np.dtype(dtype).itemsize
    lib.call(f"keydnn_cuda_add_{suf(dtype)}", da.ptr + isz, db.ptr + isz, dy.ptr + isz, n)
    assert_same_bits(dy.get()[1:], a[1:] + b[1:])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_neg_scalar_inplace_fill(oracle, dtype):
    lib = native()
    s = suf(dtype)
    for n in (5, 4099, 1 << 18):
        a, b = _inputs(n, dtype, 3)
        da, dy = Buf(lib, a), Buf(lib, shape=(n,), dtype=dtype)
        lib.call(f"keydnn_cuda_neg_{s}", da.ptr, dy.ptr, n)
        assert_same_bits(dy.get(), oracle.neg(a))
        for op, alpha in (("add", 1.5), ("sub", 0.25), ("div", 0.7), ("mul", 0.3)):
            lib.call(f"keydnn_cuda_{op}_scalar_{s}", da.ptr, cfloat(dtype, alpha), dy.ptr, n)
            assert_same_bits(dy.get(), oracle.scalar(op, a, alpha), err_msg=op)
        for op in ("gt", "ge", "lt", "le", "eq", "ne"):
            dm = Buf(lib, shape=(n,), dtype=np.float32)
            lib.call(f"keydnn_cuda_{op}_scalar_{s}", da.ptr, cfloat(dtype, 0.0), dm.ptr, n)
            np.testing.assert_array_equal(dm.get(), oracle.scalar(op, a, 0.0), err_msg=op)
        for op in ("add", "sub", "div", "mul"):
            dc, db = Buf(lib, a), Buf(lib, b)
            lib.call(f"keydnn_cuda_{op}_inplace_{s}", dc.ptr, db.ptr, n)
            assert_same_bits(dc.get(), oracle.binary(op, a, b), err_msg=op)
            dc = Buf(lib, a)
            lib.call(f"keydnn_cuda_{op}_scalar_inplace_{s}", dc.ptr, cfloat(dtype, 1.25), n)
            assert_same_bits(dc.get(), oracle.scalar(op, a, 1.25), err_msg=op)
        lib.call(f"keydnn_cuda_fill_{s}", dy.ptr, n, cfloat(dtype, -2.5))
        np.testing.assert_array_equal(dy.get(), oracle.fill(n, -2.5, dtype))
    # fill on a pointer that is not 16-byte aligned
    n = 37
    dy = Buf(lib, shape=(n + 3,), dtype=dtype, fill=0)
    isz = np.dtype(dtype).itemsize
    lib.call(f"keydnn_cuda_fill_{s}", dy.ptr + isz, n, cfloat(dtype, 3.0))
    got = dy.get()
    assert got[0] == 0 and (got[1:n + 1] == 3.0).all() and (got[n + 1:] == 0).all()


def test_status_codes_follow_the_reference():
    lib = native()
    inv_ptr = 17  # cudaErrorInvalidDevicePointer
    assert lib.raw("keydnn_cuda_add_f32")(None, None, None, 4) == inv_ptr
    assert lib.raw("keydnn_cuda_add_f32")(None, None, None, 0) == inv_ptr
    d = Buf(lib, np.zeros(4, np.float32))
    assert lib.raw("keydnn_cuda_add_f32")(d.ptr, d.ptr, d.ptr, 0) == 0
    assert lib.raw("keydnn_cuda_add_f32")(d.ptr, d.ptr, d.ptr, -5) == 0
    assert lib.raw("keydnn_cuda_mul_f32")(d.ptr, d.ptr, d.ptr, -1) == 1
    assert lib.raw("keydnn_cuda_mul_f32")(None, d.ptr, d.ptr, 4) == 2
    assert lib.raw("keydnn_cuda_mul_f32")(None, None, None, 0) == 0
    assert lib.raw("keydnn_cuda_fill_f32")(None, 4, ctypes.c_float(1)) == -1
    assert lib.raw("keydnn_cuda_fill_f32")(d.ptr, -1, ctypes.c_float(1)) == -2


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("momentum", [0.0, 0.9])
def test_sgd_step_bit_exact(oracle, dtype, momentum):
    lib = native()
    rng = np.random.default_rng(11)
    for n in (3, 1025, 25_165_824 // 64):
        p = rng.standard_normal(n).astype(dtype)
        v = np.zeros(n, dtype) if momentum else None
        dp = Buf(lib, p)
        dv = Buf(lib, v) if momentum else None
        for step in range(3):
            g = (rng.standard_normal(n) * 1e-2).astype(dtype)
            dg = Buf(lib, g)
            lib.call(f"keydnn_cuda_sgd_momentum_step_{suf(dtype)}", dp.ptr, dg.ptr, dv.ptr if dv else None, n,
                     cfloat(dtype, 0.01), cfloat(dtype, momentum), cfloat(dtype, 1e-4), cfloat(dtype, 1.0))
            p, v = oracle.sgd_step(p, g, v, 0.01, momentum, 1e-4)
            assert_same_bits(dp.get(), p, err_msg=f"step {step}")
            if momentum:
                assert_same_bits(dv.get(), v)


def test_sgd_matches_reference_golden(golden):
    lib = native()
    dp = Buf(lib, golden["sgd/p0"])
    n = dp.shape[0]
    for g, want in ((golden["sgd/g1"], golden["sgd/p1"]), (golden["sgd/g2"], golden["sgd/p2"])):
        dg = Buf(lib, g)
        lib.call("keydnn_cuda_sgd_momentum_step_f32", dp.ptr, dg.ptr, None, n, ctypes.c_float(0.01),
                 ctypes.c_float(0.0), ctypes.c_float(1e-4), ctypes.c_float(1.0))
        np.testing.assert_array_equal(dp.get(), want)


@pytest.mark.parametrize("op", ["add", "sub", "div", "gt", "ne"])
def test_same_bits_as_reference_cuda_kernels(op):
    """The reference's own kernels, compiled unmodified for sm_100a, on the same inputs."""
    ref = ref_cuda()
    if ref is None:
        pytest.skip("reference CUDA library not built")
    lib = native()
    n = (1 << 20) + 3
    a, b = _inputs(n, np.float32, 5)
    out_dt = np.float32
    outs = []
    for L in (lib, ref):
        da, db, dy = Buf(L, a), Buf(L, b), Buf(L, shape=(n,), dtype=out_dt)
        L.call(f"keydnn_cuda_{op}_f32", da.ptr, db.ptr, dy.ptr, n)
        outs.append(dy.get())
    assert_same_bits(outs[0], outs[1])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_fused_mul_div_backward_bit_exact(oracle, dtype):
    """One pass instead of the reference's two (mul) / five (div) kernels, same rounded operations."""
    lib = native()
    for n in (3, 1025, (1 << 18) + 5):
        a, b = _inputs(n, dtype, 21)
        g = np.random.default_rng(n).standard_normal(n).astype(dtype)
        dg, da, db = Buf(lib, g), Buf(lib, a), Buf(lib, b)
        for kind, want in (("mul", oracle.mul_backward(g, a, b)), ("div", oracle.div_backward(g, a, b))):
            dga, dgb = Buf(lib, shape=(n,), dtype=dtype, fill=0xFF), Buf(lib, shape=(n,), dtype=dtype, fill=0xFF)
            lib.call(f"keydnn_cuda_{kind}_backward_{suf(dtype)}", dg.ptr, da.ptr, db.ptr, dga.ptr, dgb.ptr, n)
            assert_same_bits(dga.get(), want[0].astype(dtype), err_msg=kind)
            assert_same_bits(dgb.get(), want[1].astype(dtype), err_msg=kind)
            lib.call(f"keydnn_cuda_{kind}_backward_{suf(dtype)}", dg.ptr, da.ptr, db.ptr, None, dgb.ptr, n)   # one side only
            assert_same_bits(dgb.get(), want[1].astype(dtype), err_msg=kind)
