"""Pooling through the C ABI against the CPU oracle, the golden outputs of the reference's CPU
path and the reference's own CUDA kernels.

Bars: max values / int64 argmax / routed gradients bit-exact; average pooling bit-exact where the
summation order is the reference's (the 3x3/2/1 fast path, the generic path, short-row global
average), rel 1e-5 (f32) / 1e-12 (f64) where a tree order is used (long-row global average).
"""
from __future__ import annotations

import numpy as np
import pytest

from _gpu_util import TOL, Buf, assert_same_bits, native, ref_cuda, suf

pytestmark = pytest.mark.gpu

# (N, C, H, W, k, s, p): fast paths, ragged shapes, overlap, rectangular, stride > kernel
GEOMS = [
    (2, 3, 16, 16, (2, 2), (2, 2), (0, 0)),      # 2x2/2 fast path
    (1, 2, 7, 24, (2, 2), (2, 2), (0, 0)),       # odd H: forward fast, backward generic
    (2, 2, 9, 10, (2, 2), (2, 2), (0, 0)),       # W % 8 != 0: generic
    (2, 3, 16, 24, (3, 3), (2, 2), (1, 1)),      # 3x3/2/1 avg fast path
    (1, 2, 15, 8, (3, 3), (2, 2), (1, 1)),       # odd H on the avg fast path
    (2, 2, 9, 11, (3, 3), (2, 2), (1, 1)),       # generic with padding
    (1, 3, 8, 9, (3, 2), (1, 2), (1, 0)),        # rectangular, overlapping rows
    (1, 2, 10, 10, (2, 2), (3, 3), (0, 0)),      # gaps between windows
    (3, 1, 5, 5, (5, 5), (1, 1), (2, 2)),        # window as large as the plane
    # the reference's own shape matrix (tests/infrastructure/pool2d/test_pool2d_stride_padding_shape_matrix.py)
    (2, 3, 8, 8, (2, 2), (2, 2), (0, 0)),
    (1, 1, 7, 6, (3, 2), (1, 2), (1, 0)),
    (1, 4, 9, 5, (2, 3), (2, 1), (0, 1)),
    (1, 2, 5, 5, (3, 3), (1, 1), (1, 1)),
]


def _ohw(H, W, k, s, p):
    return (H + 2 * p[0] - k[0]) // s[0] + 1, (W + 2 * p[1] - k[1]) // s[1] + 1


def _overlaps(k, s):
    return k[0] > s[0] or k[1] > s[1]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("geom", GEOMS)
def test_maxpool_ex_forward_backward(oracle, geom, dtype):
    lib = native()
    N, C, H, W, k, s, p = geom
    Ho, Wo = _ohw(H, W, k, s, p)
    rng = np.random.default_rng(H * 100 + W)
    for quant in (None, 4):                       # quantised input -> many ties
        x = rng.uniform(-1, 1, (N, C, H, W)).astype(dtype)
        if quant:
            x = (np.round(x * quant) / quant).astype(dtype)
        go = rng.standard_normal((N, C, Ho, Wo)).astype(dtype)
        y_w, idx_w = oracle.maxpool2d_forward(x, k, s, p)
        gx_w = oracle.maxpool2d_backward(go, idx_w, x.shape, p)
        dx, dgo = Buf(lib, x), Buf(lib, go)
        dy, didx = Buf(lib, shape=y_w.shape, dtype=dtype), Buf(lib, shape=y_w.shape, dtype=np.int64)
        dgx = Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF)   # must be fully overwritten
        sfx = suf(dtype)
        lib.call(f"keydnn_cuda_maxpool2d_forward_ex_{sfx}", dx.ptr, dy.ptr, didx.ptr, N, C, H, W, Ho, Wo, k[0], k[1],
                 s[0], s[1], p[0], p[1])
        np.testing.assert_array_equal(dy.get(), y_w)
        np.testing.assert_array_equal(didx.get(), idx_w)
        lib.call(f"keydnn_cuda_maxpool2d_backward_ex_{sfx}", dgo.ptr, didx.ptr, dgx.ptr, N, C, H, W, Ho, Wo, k[0],
                 k[1], s[0], s[1], p[0], p[1])
        if _overlaps(k, s):
            np.testing.assert_allclose(dgx.get(), gx_w, **TOL[np.dtype(dtype)])
        else:
            assert_same_bits(dgx.get(), gx_w)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("geom", GEOMS)
def test_avgpool_ex_forward_backward_bit_exact(oracle, geom, dtype):
    lib = native()
    N, C, H, W, k, s, p = geom
    Ho, Wo = _ohw(H, W, k, s, p)
    rng = np.random.default_rng(H * 100 + W + 1)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(dtype)
    go = rng.standard_normal((N, C, Ho, Wo)).astype(dtype)
    dx, dgo = Buf(lib, x), Buf(lib, go)
    dy = Buf(lib, shape=(N, C, Ho, Wo), dtype=dtype)
    dgx = Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF)
    sfx = suf(dtype)
    lib.call(f"keydnn_cuda_avgpool2d_forward_ex_{sfx}", dx.ptr, dy.ptr, N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1],
             p[0], p[1])
    assert_same_bits(dy.get(), oracle.avgpool2d_forward(x, k, s, p))
    lib.call(f"keydnn_cuda_avgpool2d_backward_ex_{sfx}", dgo.ptr, dgx.ptr, N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1],
             p[0], p[1])
    assert_same_bits(dgx.get(), oracle.avgpool2d_backward(go, x.shape, k, s, p))


# several bands of rows per plane, spans that start off a 16-byte boundary, windows over the edge, rows too long to stage
BAND_GEOMS = [
    (2, 3, 130, 70, (3, 3), (2, 2), (1, 1)),
    (1, 2, 200, 33, (2, 2), (2, 2), (0, 0)),
    (2, 2, 58, 58, (3, 3), (2, 2), (0, 0)),      # the padded plane of a 56x56 layer
    (1, 2, 300, 9, (5, 3), (3, 2), (2, 1)),
    (1, 3, 64, 64, (4, 4), (4, 4), (0, 0)),
    (1, 1, 12, 1500, (3, 3), (1, 1), (1, 1)),    # three rows exceed a band: the one-thread-per-element kernels
    (1, 2, 37, 41, (3, 3), (3, 3), (2, 2)),      # whole windows inside the padding
    (2, 3, 70, 60, (3, 3), (1, 1), (1, 1)),      # stride 1: three windows per axis cover an element, several bands
    (1, 2, 40, 36, (5, 4), (2, 2), (2, 1)),      # 5x4 / 2: three by two
    (2, 2, 11, 16, (2, 2), (2, 2), (0, 0)),      # the 2x2/2 kernels when aligned (odd H: a last row without a window), bands otherwise
]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("offset", [0, 1, 2, 3])
@pytest.mark.parametrize("geom", BAND_GEOMS)
def test_avgpool_row_bands_any_alignment_bit_exact(oracle, geom, offset, dtype):
    """Every tensor starts `offset` elements into its allocation; the elements in front must stay untouched."""
    lib = native()
    N, C, H, W, k, s, p = geom
    Ho, Wo = _ohw(H, W, k, s, p)
    rng = np.random.default_rng(H * 7 + W + offset)
    item = np.dtype(dtype).itemsize
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(dtype)
    go = rng.standard_normal((N, C, Ho, Wo)).astype(dtype)
    front = rng.standard_normal(offset).astype(dtype)

    def flat(a=None, n=None):
        body = a.ravel() if a is not None else np.full(n, np.nan, dtype)
        return Buf(lib, np.concatenate([front, body]))

    dx, dgo, dy, dgx = flat(x), flat(go), flat(n=go.size), flat(n=x.size)
    sfx = suf(dtype)
    at = lambda b: b.ptr + offset * item
    lib.call(f"keydnn_cuda_avgpool2d_forward_ex_{sfx}", at(dx), at(dy), N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1], p[0], p[1])
    got = dy.get()
    assert_same_bits(got[:offset], front)
    assert_same_bits(got[offset:].reshape(go.shape), oracle.avgpool2d_forward(x, k, s, p))
    lib.call(f"keydnn_cuda_avgpool2d_backward_ex_{sfx}", at(dgo), at(dgx), N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1], p[0], p[1])
    got = dgx.get()
    assert_same_bits(got[:offset], front)
    want = oracle.avgpool2d_backward(go, x.shape, k, s, p)
    assert_same_bits(got[offset:].reshape(x.shape), want)
    if p == (0, 0):
        # the reference-signature entry adds onto what the buffer holds (keydnn_avgpool2d_cuda.cu:197)
        held = rng.standard_normal(x.shape).astype(dtype)
        dacc = flat(held)
        lib.call(f"keydnn_cuda_avgpool2d_backward_{sfx}", at(dgo), at(dacc), N, C, Ho, Wo, H, W, k[0], k[1], s[0], s[1])
        got = dacc.get()
        assert_same_bits(got[:offset], front)
        assert_same_bits(got[offset:].reshape(x.shape), held + want)
        dy2 = flat(n=go.size)
        lib.call(f"keydnn_cuda_avgpool2d_forward_{sfx}", at(dx), at(dy2), N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1])
        assert_same_bits(dy2.get()[offset:].reshape(go.shape), oracle.avgpool2d_forward(x, k, s, p))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("offset", [0, 1, 2])
@pytest.mark.parametrize("geom", BAND_GEOMS)
def test_maxpool_row_bands_any_alignment(oracle, geom, offset, dtype):
    """Values and int64 positions of the banded forward kernel, ties included, on tensors that start `offset`
    elements into their allocation."""
    lib = native()
    N, C, H, W, k, s, p = geom
    Ho, Wo = _ohw(H, W, k, s, p)
    rng = np.random.default_rng(H * 11 + W + offset)
    item = np.dtype(dtype).itemsize
    x = (np.round(rng.uniform(-1, 1, (N, C, H, W)) * 8) / 8).astype(dtype)        # many ties
    x[0, 0, : min(H, 4), : min(W, 4)] = -np.inf                                     # windows without a finite tap
    x[-1, -1, H // 2, W // 2] = np.nan
    front = rng.standard_normal(offset).astype(dtype)
    dx = Buf(lib, np.concatenate([front, x.ravel()]))
    dy = Buf(lib, np.concatenate([front, np.full(N * C * Ho * Wo, np.nan, dtype)]))
    didx = Buf(lib, np.full(offset + N * C * Ho * Wo, -7, np.int64))
    sfx = suf(dtype)
    lib.call(f"keydnn_cuda_maxpool2d_forward_ex_{sfx}", dx.ptr + offset * item, dy.ptr + offset * item, didx.ptr + offset * 8,
             N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1], p[0], p[1])
    y_w, idx_w = oracle.maxpool2d_forward(x, k, s, p)
    got, got_idx = dy.get(), didx.get()
    assert_same_bits(got[:offset], front)
    np.testing.assert_array_equal(got_idx[:offset], -7)
    np.testing.assert_array_equal(got[offset:].reshape(y_w.shape), y_w)
    np.testing.assert_array_equal(got_idx[offset:].reshape(idx_w.shape), idx_w)
    # backward: every element written once; positions that point outside their window route nothing
    go = rng.standard_normal((N, C, Ho, Wo)).astype(dtype)
    idx_b = idx_w.copy()
    idx_b[0, 0, 0, 0] = -5
    idx_b[-1, -1, -1, -1] = 1 << 40
    if Ho > 2 and Wo > 2:
        idx_b[0, 0, 1, 1] = idx_w[0, 0, -1, -1]                  # inside the plane, outside its own window
    want = oracle.maxpool2d_backward(go, np.where((idx_b == idx_w), idx_w, -1), x.shape, p)
    dgo = Buf(lib, np.concatenate([front, go.ravel()]))
    didx_b = Buf(lib, np.concatenate([np.zeros(offset, np.int64), idx_b.ravel()]))
    dgx = Buf(lib, np.concatenate([front, np.full(x.size, np.nan, dtype)]))
    lib.call(f"keydnn_cuda_maxpool2d_backward_ex_{sfx}", dgo.ptr + offset * item, didx_b.ptr + offset * 8, dgx.ptr + offset * item,
             N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1], p[0], p[1])
    got = dgx.get()
    assert_same_bits(got[:offset], front)
    if _overlaps(k, s):
        np.testing.assert_allclose(got[offset:].reshape(x.shape), want, **TOL[np.dtype(dtype)])
    else:
        assert_same_bits(got[offset:].reshape(x.shape), want)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_random_geometries_against_oracle(oracle, dtype):
    """Sixty seeded random windows / strides / paddings / plane sizes (rectangular, stride larger than the window,
    windows reaching into the padding, one-pixel planes), all four pooling passes through the C ABI."""
    lib = native()
    rng = np.random.default_rng(20240521)
    sfx = suf(dtype)
    done = 0
    while done < 60:
        N, C = int(rng.integers(1, 3)), int(rng.integers(1, 4))
        H, W = int(rng.integers(1, 41)), int(rng.integers(1, 41))
        k = (int(rng.integers(1, 6)), int(rng.integers(1, 6)))
        s = (int(rng.integers(1, 5)), int(rng.integers(1, 5)))
        p = (int(rng.integers(0, k[0] // 2 + 1)), int(rng.integers(0, k[1] // 2 + 1)))
        if H + 2 * p[0] < k[0] or W + 2 * p[1] < k[1]:
            continue
        done += 1
        Ho, Wo = _ohw(H, W, k, s, p)
        x = (np.round(rng.uniform(-1, 1, (N, C, H, W)) * 16) / 16).astype(dtype)
        go = rng.standard_normal((N, C, Ho, Wo)).astype(dtype)
        tag = f"N{N} C{C} {H}x{W} k{k} s{s} p{p}"
        dx, dgo = Buf(lib, x), Buf(lib, go)
        dy, didx = Buf(lib, shape=go.shape, dtype=dtype), Buf(lib, shape=go.shape, dtype=np.int64)
        dgx = Buf(lib, shape=x.shape, dtype=dtype, fill=0xFF)
        geom = (N, C, H, W, Ho, Wo, k[0], k[1], s[0], s[1], p[0], p[1])
        lib.call(f"keydnn_cuda_avgpool2d_forward_ex_{sfx}", dx.ptr, dy.ptr, *geom)
        assert_same_bits(dy.get(), oracle.avgpool2d_forward(x, k, s, p), tag)
        lib.call(f"keydnn_cuda_avgpool2d_backward_ex_{sfx}", dgo.ptr, dgx.ptr, *geom)
        assert_same_bits(dgx.get(), oracle.avgpool2d_backward(go, x.shape, k, s, p), tag)
        lib.call(f"keydnn_cuda_maxpool2d_forward_ex_{sfx}", dx.ptr, dy.ptr, didx.ptr, *geom)
        y_w, idx_w = oracle.maxpool2d_forward(x, k, s, p)
        np.testing.assert_array_equal(dy.get(), y_w, tag)
        np.testing.assert_array_equal(didx.get(), idx_w, tag)
        lib.call(f"keydnn_cuda_maxpool2d_backward_ex_{sfx}", dgo.ptr, didx.ptr, dgx.ptr, *geom)
        want = oracle.maxpool2d_backward(go, idx_w, x.shape, p)
        if _overlaps(k, s):
            np.testing.assert_allclose(dgx.get(), want, err_msg=tag, **TOL[np.dtype(dtype)])
        else:
            assert_same_bits(dgx.get(), want, tag)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_reference_signature_entries_on_padded_planes(oracle, dtype):
    """pad2d -> pool -> (memset) -> backward -> crop2d, the reference's own call sequence
    (ops/pool2d_cuda_ext.py:56-522), gives the same results as the fused entries."""
    lib = native()
    N, C, H, W, k, s, p = 2, 3, 9, 12, (3, 3), (2, 2), (1, 1)
    Hp, Wp = H + 2 * p[0], W + 2 * p[1]
    Ho, Wo = _ohw(H, W, k, s, p)
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(dtype)
    go = rng.standard_normal((N, C, Ho, Wo)).astype(dtype)
    sfx = suf(dtype)
    from _gpu_util import cfloat
    dx, dgo = Buf(lib, x), Buf(lib, go)
    for kind, padv in (("max", -np.inf), ("avg", 0.0)):
        dxp = Buf(lib, shape=(N, C, Hp, Wp), dtype=dtype)
        lib.call(f"keydnn_cuda_pad2d_{sfx}", dx.ptr, dxp.ptr, N, C, H, W, p[0], p[1], cfloat(dtype, padv))
        np.testing.assert_array_equal(dxp.get(), oracle.pad2d(x, p[0], p[1], padv))
        dy = Buf(lib, shape=(N, C, Ho, Wo), dtype=dtype)
        dgp = Buf(lib, shape=(N, C, Hp, Wp), dtype=dtype, fill=0)
        dgx = Buf(lib, shape=x.shape, dtype=dtype)
        if kind == "max":
            didx = Buf(lib, shape=(N, C, Ho, Wo), dtype=np.int64)
            lib.call(f"keydnn_cuda_maxpool2d_forward_{sfx}", dxp.ptr, dy.ptr, didx.ptr, N, C, Hp, Wp, Ho, Wo, k[0],
                     k[1], s[0], s[1])
            y_w, idx_w = oracle.maxpool2d_forward(x, k, s, p)
            np.testing.assert_array_equal(dy.get(), y_w)
            np.testing.assert_array_equal(didx.get(), idx_w)
            lib.call(f"keydnn_cuda_maxpool2d_backward_{sfx}", dgo.ptr, didx.ptr, dgp.ptr, N, C, Ho, Wo, Hp, Wp)
            want = oracle.maxpool2d_backward(go, idx_w, x.shape, p)
        else:
            lib.call(f"keydnn_cuda_avgpool2d_forward_{sfx}", dxp.ptr, dy.ptr, N, C, Hp, Wp, Ho, Wo, k[0], k[1], s[0],
                     s[1])
            assert_same_bits(dy.get(), oracle.avgpool2d_forward(x, k, s, p))
            lib.call(f"keydnn_cuda_avgpool2d_backward_{sfx}", dgo.ptr, dgp.ptr, N, C, Ho, Wo, Hp, Wp, k[0], k[1],
                     s[0], s[1])
            want = oracle.avgpool2d_backward(go, x.shape, k, s, p)
        lib.call(f"keydnn_cuda_crop2d_{sfx}", dgp.ptr, dgx.ptr, N, C, Hp, Wp, p[0], p[1], H, W)
        np.testing.assert_allclose(dgx.get(), want, **TOL[np.dtype(dtype)])


def test_maxpool_nan_and_neg_inf_windows():
    """NaN never wins; a window of only NaN / -inf reports (-inf, window origin)  (kernel.cu:122-145)."""
    lib = native()
    x = np.zeros((1, 1, 4, 8), np.float32)
    x[0, 0, 0:2, 0:2] = np.nan
    x[0, 0, 0:2, 2:4] = -np.inf
    x[0, 0, 0:2, 4:6] = [[np.nan, 3.0], [3.0, np.nan]]
    x[0, 0, 2:4, 0:2] = [[1.0, 1.0], [1.0, 1.0]]
    dx = Buf(lib, x)
    dy, di = Buf(lib, shape=(1, 1, 2, 4), dtype=np.float32), Buf(lib, shape=(1, 1, 2, 4), dtype=np.int64)
    lib.call("keydnn_cuda_maxpool2d_forward_ex_f32", dx.ptr, dy.ptr, di.ptr, 1, 1, 4, 8, 2, 4, 2, 2, 2, 2, 0, 0)
    y, idx = dy.get()[0, 0], di.get()[0, 0]
    assert np.isneginf(y[0, 0]) and idx[0, 0] == 0
    assert np.isneginf(y[0, 1]) and idx[0, 1] == 2
    assert y[0, 2] == 3.0 and idx[0, 2] == 5          # first 3.0 in row-major order
    assert y[1, 0] == 1.0 and idx[1, 0] == 2 * 8 + 0  # tie -> first tap


def test_pool_matches_reference_golden(golden):
    lib = native()
    cases = {"k2s2p0": (2, 2, 0), "k3s2p1": (3, 2, 1), "k3s1p1": (3, 1, 1), "k2s2p0_odd": (2, 2, 0),
             "k23s21p10": ((2, 3), (2, 1), (1, 0)), "ties": (2, 2, 0)}
    pr = lambda v: (v, v) if isinstance(v, int) else v  # noqa: E731
    for name, (k, s, p) in cases.items():
        k, s, p = pr(k), pr(s), pr(p)
        x = golden[f"pool/{name}/x"]
        N, C, H, W = x.shape
        Ho, Wo = _ohw(H, W, k, s, p)
        dx = Buf(lib, x)
        dy, di = Buf(lib, shape=(N, C, Ho, Wo), dtype=np.float32), Buf(lib, shape=(N, C, Ho, Wo), dtype=np.int64)
        lib.call("keydnn_cuda_maxpool2d_forward_ex_f32", dx.ptr, dy.ptr, di.ptr, N, C, H, W, Ho, Wo, *k, *s, *p)
        np.testing.assert_array_equal(dy.get(), golden[f"pool/{name}/max_y"])
        np.testing.assert_array_equal(di.get(), golden[f"pool/{name}/max_idx"])
        go = golden.get(f"pool/{name}/max_go", np.ones((N, C, Ho, Wo), np.float32))
        dgo, dgx = Buf(lib, go), Buf(lib, shape=x.shape, dtype=np.float32)
        lib.call("keydnn_cuda_maxpool2d_backward_ex_f32", dgo.ptr, di.ptr, dgx.ptr, N, C, H, W, Ho, Wo, *k, *s, *p)
        np.testing.assert_allclose(dgx.get(), golden[f"pool/{name}/max_gx"], rtol=1e-6, atol=1e-6)
        if name == "ties":
            continue
        lib.call("keydnn_cuda_avgpool2d_forward_ex_f32", dx.ptr, dy.ptr, N, C, H, W, Ho, Wo, *k, *s, *p)
        np.testing.assert_allclose(dy.get(), golden[f"pool/{name}/avg_y"], rtol=1e-6, atol=1e-7)
        dgo = Buf(lib, golden[f"pool/{name}/avg_go"])
        lib.call("keydnn_cuda_avgpool2d_backward_ex_f32", dgo.ptr, dgx.ptr, N, C, H, W, Ho, Wo, *k, *s, *p)
        np.testing.assert_allclose(dgx.get(), golden[f"pool/{name}/avg_gx"], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape", [(3, 5, 7, 7), (2, 37, 7, 7), (4, 8, 2, 2), (2, 3, 8, 8), (2, 4, 32, 32), (1, 3, 9, 11), (3, 5, 2, 4),
                                   (2, 7, 3, 3), (5, 13, 1, 1), (64, 200, 7, 7)])
def test_global_avgpool(oracle, shape, dtype):
    lib = native()
    N, C, H, W = shape
    rng = np.random.default_rng(N * C)
    x = rng.standard_normal(shape).astype(dtype)
    go = rng.standard_normal((N, C, 1, 1)).astype(dtype)
    dx, dgo = Buf(lib, x), Buf(lib, go)
    dy, dgx = Buf(lib, shape=(N, C, 1, 1), dtype=dtype), Buf(lib, shape=shape, dtype=dtype, fill=0xFF)
    lib.call(f"keydnn_cuda_global_avgpool2d_forward_{suf(dtype)}", dx.ptr, dy.ptr, N, C, H, W)
    want = oracle.global_avgpool2d_forward(x)
    if H * W <= 64:
        assert_same_bits(dy.get(), want)          # serial (h, w) order, as the reference
    else:
        np.testing.assert_allclose(dy.get(), want, **TOL[np.dtype(dtype)])
    lib.call(f"keydnn_cuda_global_avgpool2d_backward_{suf(dtype)}", dgo.ptr, dgx.ptr, N, C, H, W)
    assert_same_bits(dgx.get(), oracle.global_avgpool2d_backward(go, shape))


def test_more_planes_than_a_grid_z_dimension(oracle):
    """N*C = 65,536 planes: the reference's gridDim.z launch cannot run this (avgpool2d_cuda.cu:219-224)."""
    lib = native()
    N, C, H, W = 256, 256, 8, 8
    rng = np.random.default_rng(9)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    dx, dy = Buf(lib, x), Buf(lib, shape=(N, C, 4, 4), dtype=np.float32)
    lib.call("keydnn_cuda_avgpool2d_forward_ex_f32", dx.ptr, dy.ptr, N, C, H, W, 4, 4, 3, 3, 2, 2, 1, 1)
    assert_same_bits(dy.get(), oracle.avgpool2d_forward(x, 3, 2, 1))


def test_same_results_as_reference_cuda_kernels(oracle):
    ref = ref_cuda()
    if ref is None:
        pytest.skip("reference CUDA library not built")
    lib = native()
    N, C, H, W, k, s = 4, 8, 32, 32, 2, 2
    rng = np.random.default_rng(21)
    x = (np.round(rng.uniform(-1, 1, (N, C, H, W)) * 8) / 8).astype(np.float32)
    go = rng.standard_normal((N, C, H // 2, W // 2)).astype(np.float32)
    res = []
    for L in (lib, ref):
        dx, dgo = Buf(L, x), Buf(L, go)
        dy, di = Buf(L, shape=go.shape, dtype=np.float32), Buf(L, shape=go.shape, dtype=np.int64)
        dgx = Buf(L, shape=x.shape, dtype=np.float32, fill=0)
        L.call("keydnn_cuda_maxpool2d_forward_f32", dx.ptr, dy.ptr, di.ptr, N, C, H, W, H // 2, W // 2, k, k, s, s)
        L.call("keydnn_cuda_maxpool2d_backward_f32", dgo.ptr, di.ptr, dgx.ptr, N, C, H // 2, W // 2, H, W)
        dya = Buf(L, shape=go.shape, dtype=np.float32)
        L.call("keydnn_cuda_avgpool2d_forward_f32", dx.ptr, dya.ptr, N, C, H, W, H // 2, W // 2, k, k, s, s)
        dg = Buf(L, shape=(N, C, 1, 1), dtype=np.float32)
        L.call("keydnn_cuda_global_avgpool2d_forward_f32", dx.ptr, dg.ptr, N, C, H, W)
        res.append((dy.get(), di.get(), dgx.get(), dya.get(), dg.get()))
    (y0, i0, g0, a0, p0), (y1, i1, g1, a1, p1) = res
    np.testing.assert_array_equal(y0, y1)
    np.testing.assert_array_equal(i0, i1)
    assert_same_bits(g0, g1)
    assert_same_bits(a0, a1)
    np.testing.assert_allclose(p0, p1, rtol=1e-5, atol=1e-6)


def test_maxpool_padding_never_wins_and_gradient_stays_in_bounds():
    """The reference's padding trap (tests/infrastructure/pool2d/test_maxpool2d_padding_trap.py): strictly negative
    input, windows that reach into the padding; padding must behave as -inf, so every output is a real (negative)
    input and every upstream gradient lands on a real input."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import pooling

    x = np.array([[[[-1.0, -2.0], [-3.0, -4.0]]]], dtype=np.float32)
    tx = kd.Tensor.from_numpy(x, requires_grad=True)
    y = pooling.MaxPool2d(kernel_size=(2, 2), stride=(1, 1), padding=(1, 1))(tx)
    assert y.shape == (1, 1, 3, 3)
    yv = y.to_numpy()
    assert (yv < 0).all(), yv
    np.testing.assert_array_equal(yv[0, 0], [[-1, -1, -2], [-1, -1, -2], [-3, -3, -4]])
    y.backward(kd.Tensor.ones(y.shape))
    gx = tx.grad.to_numpy()
    assert np.isfinite(gx).all() and gx.sum() == 9.0
    np.testing.assert_array_equal(gx[0, 0], [[4, 2], [2, 1]])
