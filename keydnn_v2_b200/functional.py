"""Activation Functions and modules, the loss Functions, and Adam, on CUDA tensors.

Host-side mirror of
  * ``src/keydnn/infrastructure/_function.py:54-612`` (``ExpFn`` / ``SigmoidFn`` / ``ReLUFn`` /
    ``LeakyReLUFn`` / ``TanhFn`` / ``SoftmaxFn``: static ``forward(ctx, x, ...)`` / ``backward(ctx, grad_out)``,
    and the ``exp`` helper),
  * ``_activations.py:44-325`` (``Sigmoid`` / ``ReLU`` / ``LeakyReLU`` / ``Tanh`` / ``Softmax`` modules),
  * ``_losses.py:44-408`` (``SSEFn`` / ``MSEFn`` / ``BinaryCrossEntropyFn`` / ``CategoricalCrossEntropyFn``),
  * ``optimizers/_adam.py:60-220`` (``Adam``: same constructor checks; its ``step`` raises for CUDA
    parameters in the reference).

Where the reference chains one-op tensor kernels with a temporary between each pair, every forward
and every backward here is one launch of a fused kernel that applies the same separately rounded
operations, so values are the reference's own.  No loss backward reads the upstream scalar to the
host (the reference calls ``item()``): the device scalar is passed to the kernel.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .tensor import Context, Parameter, Tensor, _suffix, no_grad


def _call(x: Tensor, name: str, *args) -> None:
    x.native.call(f"keydnn_cuda_{name}_{_suffix(x.dtype)}", *args)


def _scalar_arg(x: Tensor, v: float):
    return ctypes.c_float(v) if x.dtype == np.float32 else ctypes.c_double(v)


def _unary(name: str, x: Tensor, *extra) -> Tensor:
    y = Tensor.empty(x.shape, x.dtype)
    if x.numel:
        _call(x, name, x.data, y.data, *extra, x.numel)
    return y


def _binary(name: str, a: Tensor, b: Tensor, *extra) -> Tensor:
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError(f"{name}: shape / dtype mismatch {a.shape} {a.dtype} vs {b.shape} {b.dtype}")
    y = Tensor.empty(a.shape, a.dtype)
    if a.numel:
        _call(a, name, a.data, b.data, y.data, *extra, a.numel)
    return y


# ---------------------------------------------------------------------------
# Functions
# ---------------------------------------------------------------------------
class ExpFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor) -> Tensor:
        if x.numel > 0x7FFFFFFF:
            raise ValueError("exp: the reference entry takes a 32-bit element count")
        out = _unary("exp", x)
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor) -> Tensor:
        (out,) = ctx.saved_tensors
        with no_grad():
            return grad_out * out


class SigmoidFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor) -> Tensor:
        out = _unary("sigmoid_forward", x)
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor) -> Tensor:
        (out,) = ctx.saved_tensors
        return _binary("sigmoid_backward", grad_out, out)


class ReLUFn:
    """Saves the input instead of the reference's float mask (same bytes kept alive, one kernel fewer)."""

    @staticmethod
    def forward(ctx: Context, x: Tensor) -> Tensor:
        y = Tensor.empty(x.shape, x.dtype)
        if x.numel:
            _call(x, "relu_forward", x.data, y.data, None, x.numel)
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor) -> Tensor:
        (x,) = ctx.saved_tensors
        return _binary("relu_backward", grad_out, x)


class LeakyReLUFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor, alpha: float = 0.01) -> Tensor:
        ctx.save_for_backward(x)
        ctx.saved_meta["alpha"] = float(alpha)
        return _unary("leaky_relu_forward", x, _scalar_arg(x, float(alpha)))

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor) -> Tensor:
        (x,) = ctx.saved_tensors
        return _binary("leaky_relu_backward", grad_out, x, _scalar_arg(x, float(ctx.saved_meta["alpha"])))


class TanhFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor) -> Tensor:
        out = _unary("tanh_forward", x)
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor) -> Tensor:
        (out,) = ctx.saved_tensors
        return _binary("tanh_backward", grad_out, out)


def _axis_view(shape: Sequence[int], axis: int) -> Tuple[int, int, int]:
    outer = int(np.prod(shape[:axis], dtype=np.int64))
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
    return outer, int(shape[axis]), inner


class SoftmaxFn:
    @staticmethod
    def forward(ctx: Context, x: Tensor, *, axis: int = -1) -> Tensor:
        ndim = len(x.shape)
        axis_ = axis if axis >= 0 else ndim + axis
        if axis_ < 0 or axis_ >= ndim:
            raise ValueError(f"Invalid softmax axis {axis} for ndim={ndim}")
        y = Tensor.empty(x.shape, x.dtype)
        if x.numel:
            _call(x, "softmax_forward", x.data, y.data, *_axis_view(x.shape, axis_))
        ctx.save_for_backward(y)
        ctx.saved_meta["axis"] = axis_
        return y

    @staticmethod
    def backward(ctx: Context, grad_out: Tensor) -> Tuple[Tensor]:
        (y,) = ctx.saved_tensors
        if grad_out.shape != y.shape or grad_out.dtype != y.dtype:
            raise ValueError("softmax backward: grad_out must match the output")
        dx = Tensor.empty(y.shape, y.dtype)
        if y.numel:
            _call(y, "softmax_backward", grad_out.data, y.data, dx.data, *_axis_view(y.shape, int(ctx.saved_meta["axis"])))
        return (dx,)


def _apply(fn, x: Tensor, **kw) -> Tensor:
    """Run ``fn.forward`` and, when ``x`` is in the graph, attach a node that calls ``fn.backward``.
    The node's closure holds the saved state, not the node, so no reference cycle keeps activations alive."""
    saved = Context((x,), None)
    y = fn.forward(saved, x, **kw)
    if x._needs_grad():
        y.requires_grad = True

        def backward_fn(g: Tensor):
            r = fn.backward(saved, g)
            return r if isinstance(r, tuple) else (r,)

        y._set_ctx(Context((x,), backward_fn))
    return y


def exp(x: Tensor) -> Tensor:
    """``_function.py:118-156``."""
    return _apply(ExpFn, x)


def log(x: Tensor) -> Tensor:
    """``tensor/mixins/unary/_tensor_log.py:60-123``: y = log(x); backward grad_out / x.  On the device (the
    reference copies the tensor to the host and back)."""
    y = _unary("log", x)
    if x._needs_grad():
        y.requires_grad = True

        def backward_fn(g: Tensor):
            with no_grad():
                return (g / x,)

        y._set_ctx(Context((x,), backward_fn))
    return y


def sqrt(x: Tensor) -> Tensor:
    """``tensor/mixins/unary/_tensor_sqrt.py:60-125``: backward grad_out * (0.5 / out), one kernel."""
    y = _unary("sqrt", x)
    if x._needs_grad():
        y.requires_grad = True
        out = y.detach()
        y._set_ctx(Context((x,), lambda g: (_binary("sqrt_backward", g, out),)))
    return y


def sigmoid(x: Tensor) -> Tensor:
    return _apply(SigmoidFn, x)


def relu(x: Tensor) -> Tensor:
    return _apply(ReLUFn, x)


def leaky_relu(x: Tensor, alpha: float = 0.01) -> Tensor:
    return _apply(LeakyReLUFn, x, alpha=alpha)


def tanh(x: Tensor) -> Tensor:
    return _apply(TanhFn, x)


def softmax(x: Tensor, axis: int = -1) -> Tensor:
    return _apply(SoftmaxFn, x, axis=axis)


# ---------------------------------------------------------------------------
# Modules (_activations.py)
# ---------------------------------------------------------------------------
class _Stateless:
    def __call__(self, x: Tensor) -> Tensor:
        return self.forward(x)

    def parameters(self) -> List[Parameter]:
        return []


class Sigmoid(_Stateless):
    def forward(self, x: Tensor) -> Tensor:
        return sigmoid(x)


class ReLU(_Stateless):
    def forward(self, x: Tensor) -> Tensor:
        return relu(x)


class LeakyReLU(_Stateless):
    def __init__(self, alpha: float = 0.01) -> None:
        self.alpha = float(alpha)

    def forward(self, x: Tensor) -> Tensor:
        return leaky_relu(x, self.alpha)


class Tanh(_Stateless):
    def forward(self, x: Tensor) -> Tensor:
        return tanh(x)


class Softmax(_Stateless):
    def __init__(self, *, axis: int = -1) -> None:
        self._axis = axis

    def forward(self, x: Tensor) -> Tensor:
        return softmax(x, self._axis)


# ---------------------------------------------------------------------------
# Losses (_losses.py).  Functions keep the reference's forward(ctx, pred, target) /
# backward(ctx, grad_out) shape; grad_out is the scalar upstream gradient tensor (or None = 1).
# ---------------------------------------------------------------------------
def _check_pair(pred: Tensor, target: Tensor, what: str) -> None:
    if pred.shape != target.shape or pred.dtype != target.dtype:
        raise ValueError(f"{what}: pred and target must have the same shape and dtype, got {pred.shape} {pred.dtype} "
                         f"and {target.shape} {target.dtype}")
    if pred.numel == 0:
        raise ValueError(f"{what}: empty input")


def _g_ptr(grad_out: Optional[Tensor]):
    if grad_out is None or getattr(grad_out, "_is_unit_seed", False):
        return None
    if grad_out.numel != 1:
        raise ValueError("the upstream gradient of a loss is a scalar")
    return grad_out.data


class _SqDiffFn:
    MEAN = 0

    @classmethod
    def forward(cls, ctx: Context, pred: Tensor, target: Tensor) -> Tensor:
        _check_pair(pred, target, cls.__name__)
        diff = Tensor.empty(pred.shape, pred.dtype)
        loss = Tensor.empty((), pred.dtype)
        _call(pred, "sqdiff_forward", pred.data, target.data, diff.data, loss.data, pred.numel, cls.MEAN)
        ctx.save_for_backward(diff)
        ctx.saved_meta["n"] = pred.numel
        return loss

    @classmethod
    def backward(cls, ctx: Context, grad_out: Optional[Tensor], *, need_target_grad: bool = True):
        (diff,) = ctx.saved_tensors
        n = int(ctx.saved_meta["n"])
        scale = (2.0 / n) if cls.MEAN else 2.0
        gp = Tensor.empty(diff.shape, diff.dtype)
        gt = Tensor.empty(diff.shape, diff.dtype) if need_target_grad else None
        _call(diff, "sqdiff_backward", diff.data, _g_ptr(grad_out), ctypes.c_double(scale), gp.data,
              gt.data if gt is not None else None, n)
        return gp, gt


class SSEFn(_SqDiffFn):
    """``_losses.py:44-127``: sum((pred - target)^2); gradients 2*g*diff and its negative."""
    MEAN = 0


class MSEFn(_SqDiffFn):
    """``_losses.py:130-216``: mean((pred - target)^2); gradients ((2/n)*g)*diff and its negative."""
    MEAN = 1


class BinaryCrossEntropyFn:
    """``_losses.py:219-317``."""

    @staticmethod
    def forward(ctx: Context, pred: Tensor, target: Tensor) -> Tensor:
        _check_pair(pred, target, "BinaryCrossEntropyFn")
        ctx.save_for_backward(pred, target)
        ctx.saved_meta["n"] = pred.numel
        loss = Tensor.empty((), pred.dtype)
        _call(pred, "bce_forward", pred.data, target.data, loss.data, pred.numel)
        return loss

    @staticmethod
    def backward(ctx: Context, grad_out: Optional[Tensor]):
        pred, target = ctx.saved_tensors
        gp = Tensor.empty(pred.shape, pred.dtype)
        _call(pred, "bce_backward", pred.data, target.data, _g_ptr(grad_out), gp.data, pred.numel)
        return gp, None


class CategoricalCrossEntropyFn:
    """``_losses.py:320-408``: pred (N, C) probabilities, target one-hot; mean over the batch."""

    @staticmethod
    def forward(ctx: Context, pred: Tensor, target: Tensor) -> Tensor:
        _check_pair(pred, target, "CategoricalCrossEntropyFn")
        ctx.save_for_backward(pred, target)
        loss = Tensor.empty((), pred.dtype)
        _call(pred, "cce_forward", pred.data, target.data, loss.data, pred.numel, pred.shape[0])
        return loss

    @staticmethod
    def backward(ctx: Context, grad_out: Optional[Tensor]):
        pred, target = ctx.saved_tensors
        gp = Tensor.empty(pred.shape, pred.dtype)
        _call(pred, "cce_backward", pred.data, target.data, _g_ptr(grad_out), gp.data, pred.numel, pred.shape[0])
        return gp, None


def _loss(fn, pred: Tensor, target: Tensor) -> Tensor:
    saved = Context((pred, target), None)
    loss = fn.forward(saved, pred, target)
    need_p, need_t = pred._needs_grad(), target._needs_grad()
    if need_p or need_t:
        loss.requires_grad = True

        def backward_fn(g: Tensor):
            if issubclass(fn, _SqDiffFn):
                gp, gt = fn.backward(saved, g, need_target_grad=need_t)
            else:
                gp, gt = fn.backward(saved, g)
            return (gp if need_p else None, gt if need_t else None)

        loss._set_ctx(Context((pred, target), backward_fn))
    return loss


def sse_loss(pred: Tensor, target: Tensor) -> Tensor:
    return _loss(SSEFn, pred, target)


def mse_loss(pred: Tensor, target: Tensor) -> Tensor:
    return _loss(MSEFn, pred, target)


def binary_cross_entropy(pred: Tensor, target: Tensor) -> Tensor:
    return _loss(BinaryCrossEntropyFn, pred, target)


def categorical_cross_entropy(pred: Tensor, target: Tensor) -> Tensor:
    return _loss(CategoricalCrossEntropyFn, pred, target)


# ---------------------------------------------------------------------------
# Adam (optimizers/_adam.py)
# ---------------------------------------------------------------------------
class Adam:
    """Adam with coupled L2 weight decay.  Constructor checks as ``optimizers/_adam.py:120-139``; the update
    of ``:190-219`` (eleven tensor passes and as many temporaries per parameter on the CPU, a
    device-not-supported error on CUDA) is one in-place kernel per parameter here, with the per-step
    scalars ``1 - beta^t`` formed in Python doubles as the reference forms them."""

    def __init__(self, params: Iterable[Parameter], lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0) -> None:
        self.params = list(params)
        self.lr = float(lr)
        self.betas = (float(betas[0]), float(betas[1]))
        self.eps = float(eps)
        self.weight_decay = float(weight_decay)
        b1, b2 = self.betas
        if self.lr <= 0.0:
            raise ValueError(f"lr must be > 0, got {self.lr}")
        if not (0.0 < b1 < 1.0) or not (0.0 < b2 < 1.0):
            raise ValueError(f"betas must be in (0,1), got {self.betas}")
        if self.eps <= 0.0:
            raise ValueError(f"eps must be > 0, got {self.eps}")
        if self.weight_decay < 0.0:
            raise ValueError(f"weight_decay must be >= 0, got {self.weight_decay}")
        self._state = {}

    def zero_grad(self) -> None:
        for p in self.params:
            p.zero_grad()

    def step(self) -> None:
        b1, b2 = self.betas
        for p in self.params:
            g = p.grad
            if g is None:
                continue
            st = self._state.get(id(p))
            if st is None:
                st = {"t": 0, "m": Tensor.zeros(p.shape, p.dtype), "v": Tensor.zeros(p.shape, p.dtype)}
                self._state[id(p)] = st
            st["t"] += 1
            t = st["t"]
            c = lambda v: _scalar_arg(p, v)   # noqa: E731
            _call(p, "adam_step", p.data, g.data, st["m"].data, st["v"].data, p.numel, c(self.lr), c(b1), c(b2), c(self.eps),
                  c(self.weight_decay), c(1.0 - b1), c(1.0 - b2), c(1.0 - b1 ** t), c(1.0 - b2 ** t), c(1.0))
