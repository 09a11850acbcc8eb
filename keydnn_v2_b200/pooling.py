"""Pooling on CUDA tensors: ext-level functions, autograd Functions and Modules.

Host-side mirror of
  * ``src/keydnn/infrastructure/ops/pool2d_cuda_ext.py:56-620`` (``maxpool2d_forward`` ...
    ``global_avgpool2d_backward``: same names, keyword arguments and return values), and
  * ``src/keydnn/infrastructure/pooling/_pooling_function.py:62-384`` /
    ``_pooling_module.py:74-372`` (``MaxPool2dFn`` / ``AvgPool2dFn`` / ``GlobalAvgPool2dFn``
    and the ``MaxPool2d`` / ``AvgPool2d`` / ``GlobalAvgPool2d`` modules).

Where the reference runs pad2d -> pool (forward) and memset -> pool-backward -> crop2d
(backward) with a device synchronisation after each step, these call the fused
``*_ex`` entries of the library once and do not synchronise.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import numpy as np

from ._cuda_storage import CudaStorage
from .tensor import Context, Tensor, _suffix

IntPair = Union[int, Tuple[int, int]]


def _pair(v: IntPair) -> Tuple[int, int]:
    if isinstance(v, int):
        return (v, v)
    if len(v) != 2:
        raise ValueError(f"expected an int or a pair, got {v!r}")
    return (int(v[0]), int(v[1]))


def _out_hw(H: int, W: int, k, s, p) -> Tuple[int, int]:
    H_out = (H + 2 * p[0] - k[0]) // s[0] + 1
    W_out = (W + 2 * p[1] - k[1]) // s[1] + 1
    if H_out <= 0 or W_out <= 0:
        raise ValueError(f"pooling window {k} with stride {s}, padding {p} does not fit input {(H, W)}")
    return H_out, W_out


def _require_cuda_4d(x: Tensor, name: str) -> None:
    if not isinstance(x, Tensor):
        raise TypeError(f"{name} must be a CUDA Tensor")
    if x.ndim != 4:
        raise ValueError(f"{name} must be NCHW (4-D), got shape {x.shape}")
    _suffix(x.dtype)


# ---------------------------------------------------------------------------
# ext level
# ---------------------------------------------------------------------------
def maxpool2d_forward(x: Tensor, *, kernel_size: IntPair, stride: Optional[IntPair] = None, padding: IntPair = 0,
                      device: int = 0) -> Tuple[Tensor, CudaStorage]:
    """Returns ``(y, argmax_idx_storage)``; the int64 positions are ``h*W_pad + w`` in the padded plane."""
    _require_cuda_4d(x, "x")
    k, s, p = _pair(kernel_size), _pair(kernel_size if stride is None else stride), _pair(padding)
    N, C, H, W = x.shape
    H_out, W_out = _out_hw(H, W, k, s, p)
    y = Tensor.empty((N, C, H_out, W_out), x.dtype)
    idx = CudaStorage.allocate(N * C * H_out * W_out * 8, np.int64)
    x.native.call(f"keydnn_cuda_maxpool2d_forward_ex_{_suffix(x.dtype)}", x.data, y.data, idx.dev_ptr, N, C, H, W,
                  H_out, W_out, k[0], k[1], s[0], s[1], p[0], p[1])
    return y, idx


def maxpool2d_backward(grad_out: Tensor, *, argmax_idx, x_shape: Sequence[int], kernel_size: IntPair,
                       stride: IntPair, padding: IntPair, device: int = 0) -> Tensor:
    _require_cuda_4d(grad_out, "grad_out")
    k, s, p = _pair(kernel_size), _pair(stride), _pair(padding)
    N, C, H, W = (int(d) for d in x_shape)
    H_out, W_out = grad_out.shape[2], grad_out.shape[3]
    gx = Tensor.empty((N, C, H, W), grad_out.dtype)
    grad_out.native.call(f"keydnn_cuda_maxpool2d_backward_ex_{_suffix(grad_out.dtype)}", grad_out.data,
                         int(argmax_idx), gx.data, N, C, H, W, H_out, W_out, k[0], k[1], s[0], s[1], p[0], p[1])
    return gx


def avgpool2d_forward(x: Tensor, *, kernel_size: IntPair, stride: Optional[IntPair] = None, padding: IntPair = 0,
                      device: int = 0) -> Tensor:
    _require_cuda_4d(x, "x")
    k, s, p = _pair(kernel_size), _pair(kernel_size if stride is None else stride), _pair(padding)
    N, C, H, W = x.shape
    H_out, W_out = _out_hw(H, W, k, s, p)
    y = Tensor.empty((N, C, H_out, W_out), x.dtype)
    x.native.call(f"keydnn_cuda_avgpool2d_forward_ex_{_suffix(x.dtype)}", x.data, y.data, N, C, H, W, H_out, W_out,
                  k[0], k[1], s[0], s[1], p[0], p[1])
    return y


def avgpool2d_backward(grad_out: Tensor, *, x_shape: Sequence[int], kernel_size: IntPair, stride: IntPair,
                       padding: IntPair, device: int = 0) -> Tensor:
    _require_cuda_4d(grad_out, "grad_out")
    k, s, p = _pair(kernel_size), _pair(stride), _pair(padding)
    N, C, H, W = (int(d) for d in x_shape)
    H_out, W_out = grad_out.shape[2], grad_out.shape[3]
    gx = Tensor.empty((N, C, H, W), grad_out.dtype)
    grad_out.native.call(f"keydnn_cuda_avgpool2d_backward_ex_{_suffix(grad_out.dtype)}", grad_out.data, gx.data, N,
                         C, H, W, H_out, W_out, k[0], k[1], s[0], s[1], p[0], p[1])
    return gx


def global_avgpool2d_forward(x: Tensor, *, device: int = 0) -> Tensor:
    _require_cuda_4d(x, "x")
    N, C, H, W = x.shape
    y = Tensor.empty((N, C, 1, 1), x.dtype)
    x.native.call(f"keydnn_cuda_global_avgpool2d_forward_{_suffix(x.dtype)}", x.data, y.data, N, C, H, W)
    return y


def global_avgpool2d_backward(grad_out: Tensor, *, x_shape: Sequence[int], device: int = 0) -> Tensor:
    _require_cuda_4d(grad_out, "grad_out")
    N, C, H, W = (int(d) for d in x_shape)
    if grad_out.shape != (N, C, 1, 1):
        raise ValueError(f"grad_out must have shape {(N, C, 1, 1)}, got {grad_out.shape}")
    gx = Tensor.empty((N, C, H, W), grad_out.dtype)
    grad_out.native.call(f"keydnn_cuda_global_avgpool2d_backward_{_suffix(grad_out.dtype)}", grad_out.data, gx.data,
                         N, C, H, W)
    return gx


# ---------------------------------------------------------------------------
# autograd Functions (static forward(ctx, ...) / backward(ctx, grad_out))
# ---------------------------------------------------------------------------
class MaxPool2dFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor, *, kernel_size: IntPair, stride: Optional[IntPair] = None,
                padding: IntPair = 0) -> Tensor:
        k, s, p = _pair(kernel_size), _pair(kernel_size if stride is None else stride), _pair(padding)
        y, idx = maxpool2d_forward(x, kernel_size=k, stride=s, padding=p)
        ctx.saved_meta.update(x_shape=x.shape, kernel_size=k, stride=s, padding=p, argmax_idx=idx)
        return y

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor):
        m = ctx.saved_meta
        return (maxpool2d_backward(grad_out, argmax_idx=m["argmax_idx"], x_shape=m["x_shape"],
                                   kernel_size=m["kernel_size"], stride=m["stride"], padding=m["padding"]),)


class AvgPool2dFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor, *, kernel_size: IntPair, stride: Optional[IntPair] = None,
                padding: IntPair = 0) -> Tensor:
        k, s, p = _pair(kernel_size), _pair(kernel_size if stride is None else stride), _pair(padding)
        ctx.saved_meta.update(x_shape=x.shape, kernel_size=k, stride=s, padding=p)
        return avgpool2d_forward(x, kernel_size=k, stride=s, padding=p)

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor):
        m = ctx.saved_meta
        return (avgpool2d_backward(grad_out, x_shape=m["x_shape"], kernel_size=m["kernel_size"], stride=m["stride"],
                                   padding=m["padding"]),)


class GlobalAvgPool2dFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor) -> Tensor:
        ctx.saved_meta.update(x_shape=x.shape)
        return global_avgpool2d_forward(x)

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor):
        return (global_avgpool2d_backward(grad_out, x_shape=ctx.saved_meta["x_shape"]),)


def _apply(fn, x: Tensor, **kw) -> Tensor:
    # `saved` is what forward fills and backward reads.  The graph node's closure refers to it, not
    # to the node itself, so the node is not part of a reference cycle and its activations are
    # released by reference counting as soon as the graph is dropped (the reference's modules close
    # over their own Context, pooling/_pooling_module.py:183-198, and wait for the cyclic collector).
    saved = Context((x,), None)
    y = fn.forward(saved, x, **kw)
    if x._needs_grad():
        y.requires_grad = True
        node = Context((x,), lambda g: fn.backward(saved, g))
        node.saved_meta = saved.saved_meta
        y._set_ctx(node)
    return y


# ---------------------------------------------------------------------------
# Modules
# ---------------------------------------------------------------------------
class MaxPool2d:
    def __init__(self, kernel_size: IntPair, stride: Optional[IntPair] = None, padding: IntPair = 0) -> None:
        self.kernel_size = _pair(kernel_size)
        self.stride = _pair(kernel_size if stride is None else stride)
        self.padding = _pair(padding)

    def forward(self, x: Tensor) -> Tensor:
        return _apply(MaxPool2dFn, x, kernel_size=self.kernel_size, stride=self.stride, padding=self.padding)

    __call__ = forward

    def parameters(self):
        return []


class AvgPool2d(MaxPool2d):
    def forward(self, x: Tensor) -> Tensor:
        return _apply(AvgPool2dFn, x, kernel_size=self.kernel_size, stride=self.stride, padding=self.padding)

    __call__ = forward


class GlobalAvgPool2d:
    def forward(self, x: Tensor) -> Tensor:
        return _apply(GlobalAvgPool2dFn, x)

    __call__ = forward

    def parameters(self):
        return []
