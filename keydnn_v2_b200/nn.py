"""Layers, loss and optimizer of the small-CNN training step, on CUDA tensors.

Host-side mirror of the reference modules that surround the pool / reduce / elementwise path in a
CNN layer stack (paths under ``src/keydnn/infrastructure/``):
  ``convolution/_conv2d_module.py`` + ``_conv2d_function.py``   Conv2d (cuDNN, kept a library call)
  ``layers/_batchnorm.py:430-700``                              BatchNorm2d (CPU-only in the reference)
  ``_activations.py`` / ``_function.py:291-293``                ReLU = (x > 0) mask, x * mask
  ``flatten/``, ``fully_connected/_linear.py:283-291``          Flatten, Linear (cuBLAS + bias_add)
  ``_losses.py:150-215``                                        MSE = mean((pred - target)^2)
  ``optimizers/_sgd.py:119-140``                                SGD with coupled weight decay
  ``models/_sequential.py:130-152``                             Sequential

Same constructor arguments, parameter shapes, initialisers (NumPy global RNG, Kaiming normal =
randn * sqrt(2 / fan_in), zeros for biases) and formulas.  What differs is where the work runs:
everything stays on the device (no host round trip around cuDNN, no host sqrt in BatchNorm), the
optimizer updates all parameters with one fused kernel over a flat buffer, and momentum (absent in
the reference optimizer) is available.
"""
from __future__ import annotations

import ctypes
import math
from typing import Iterable, List, Sequence, Tuple

import numpy as np

from ._cuda_storage import CudaStorage
from ._native import load_dnn
from .pooling import GlobalAvgPool2d, MaxPool2d, _pair  # noqa: F401  (re-exported for model code)
from .tensor import Context, Parameter, Tensor, _suffix, no_grad


def _cfloat(dtype, v: float):
    return ctypes.c_float(v) if np.dtype(dtype) == np.float32 else ctypes.c_double(v)


class Module:
    training = True

    def parameters(self) -> List[Parameter]:
        out: List[Parameter] = []
        for v in self.__dict__.values():
            if isinstance(v, Parameter):
                out.append(v)
            elif isinstance(v, Module):
                out.extend(v.parameters())
            elif isinstance(v, (list, tuple)):
                for m in v:
                    if isinstance(m, Module):
                        out.extend(m.parameters())
                    elif hasattr(m, "parameters") and not isinstance(m, Tensor):
                        out.extend(m.parameters())
        return out

    def train(self, mode: bool = True) -> "Module":
        self.training = mode
        for v in self.__dict__.values():
            if isinstance(v, Module):
                v.train(mode)
            elif isinstance(v, (list, tuple)):
                for m in v:
                    if isinstance(m, Module):
                        m.train(mode)
        return self

    def eval(self) -> "Module":
        return self.train(False)

    def __call__(self, *a, **k):
        return self.forward(*a, **k)


def kaiming_normal(shape: Sequence[int], dtype=np.float32) -> np.ndarray:
    """``utils/weight_initializer/_kaiming.py:55-63``: randn(*shape) * sqrt(2 / fan_in) from the global NumPy RNG;
    fan_in = in_features for (out, in), C_in * K_h * K_w for (C_out, C_in, K_h, K_w)."""
    fan_in = int(np.prod(shape[1:])) if len(shape) > 1 else int(shape[0])
    return np.random.randn(*shape).astype(dtype, copy=False) * dtype(math.sqrt(2.0 / float(max(1, fan_in))))


class Conv2d(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, bias: bool = True,
                 dtype=np.float32, initializer: str = "kaiming") -> None:
        if initializer != "kaiming":
            raise ValueError("only the reference default initializer 'kaiming' is implemented")
        self.in_channels, self.out_channels = int(in_channels), int(out_channels)
        self.kernel_size, self.stride, self.padding = _pair(kernel_size), _pair(stride), _pair(padding)
        self.weight = Parameter.from_numpy(kaiming_normal((out_channels, in_channels, *self.kernel_size), np.dtype(dtype).type))
        self.bias = Parameter.from_numpy(np.zeros(out_channels, dtype)) if bias else None
        self.bias_deferred = False      # set by Sequential when a BatchNorm2d follows: that layer adds the bias as it reads

    def forward(self, x: Tensor) -> Tensor:
        if x.ndim != 4 or x.shape[1] != self.in_channels:
            raise ValueError(f"Conv2d expects (N, {self.in_channels}, H, W), got {x.shape}")
        dnn = load_dnn()
        N, C, H, W = x.shape
        (kh, kw), (sh, sw), (ph, pw) = self.kernel_size, self.stride, self.padding
        Ho, Wo = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        s = _suffix(x.dtype)
        y = Tensor.empty((N, self.out_channels, Ho, Wo), x.dtype)
        dims = (N, C, H, W, self.out_channels, Ho, Wo, kh, kw, sh, sw, ph, pw)
        dnn.call(f"keydnn_cuda_conv2d_forward_ex_{s}", x.data, self.weight.data,
                 self.bias.data if self.bias and not self.bias_deferred else None, y.data, *dims)
        w, b = self.weight, self.bias
        if x._needs_grad(w) or (b is not None and b.requires_grad):
            y.requires_grad = True

            def backward_fn(g: Tensor):
                gx = Tensor.empty(x.shape, x.dtype) if x.requires_grad else None
                gw = w.grad_buffer()
                dnn.call(f"keydnn_cuda_conv2d_backward_ex_{s}", x.data, w.data, g.data, gx.data if gx else None, gw.data,
                         *dims)
                if b is None:
                    return (gx, gw)
                with no_grad():     # the reference sums the bias gradient on the host (ops/conv2d_cuda.py:573-575)
                    gb = g.sum_to_shape((1, self.out_channels, 1, 1)).reshape(self.out_channels)
                return (gx, gw, gb)

            y._ctx = Context((x, w) if b is None else (x, w, b), backward_fn)
        return y


class BatchNorm2d(Module):
    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 dtype=np.float32) -> None:
        self.num_features, self.eps, self.momentum, self.affine = int(num_features), float(eps), float(momentum), affine
        self.gamma = Parameter.from_numpy(np.ones(num_features, dtype)) if affine else None
        self.beta = Parameter.from_numpy(np.zeros(num_features, dtype)) if affine else None
        self.running_mean = Tensor.zeros((num_features,), dtype)
        self.running_var = Tensor.ones((num_features,), dtype)
        self.fused_relu = False     # set by Sequential when a ReLU follows: one kernel pair does both layers
        self.pre_bias = None        # set by Sequential when a Conv2d precedes: its bias, added while x is read
        self.fused_pool = None      # set by Sequential when a MaxPool2d(2) follows: pooled in the same pass
        self.fused_gap = None       # set by Sequential when a GlobalAvgPool2d follows: averaged in the same pass

    def parameters(self) -> List[Parameter]:
        return [self.gamma, self.beta] if self.affine else []

    def forward(self, x: Tensor) -> Tensor:
        if x.ndim != 4:
            raise ValueError(f"BatchNorm2d expects 4D input (N, C, H, W), got shape {x.shape}")
        N, C, H, W = x.shape
        if C != self.num_features:
            raise ValueError(f"Expected num_features={self.num_features}, got C={C}")
        lib, s = x.native, _suffix(x.dtype)
        mean, invstd = Tensor.empty((C,), x.dtype), Tensor.empty((C,), x.dtype)
        ga, be = (self.gamma, self.beta) if self.affine else (None, None)
        pb = self.pre_bias
        if self.fused_pool is not None and H % 2 == 0 and W % 8 == 0 and N * C * H * W < (1 << 34):
            return self._forward_pooled(x, mean, invstd, ga, be, pb)
        if self.fused_gap is not None and (H * W) % 4 == 0 and 64 < H * W < (1 << 31):
            return self._forward_averaged(x, mean, invstd, ga, be, pb)
        y = Tensor.empty(x.shape, x.dtype)
        lib.call(f"keydnn_cuda_bn2d_forward_bias_{s}", x.data, pb.data if pb is not None else None, ga.data if ga else None,
                 be.data if be else None, y.data, mean.data, invstd.data, self.running_mean.data, self.running_var.data,
                 N, C, H * W, _cfloat(x.dtype, self.eps), _cfloat(x.dtype, self.momentum), 1 if self.training else 0,
                 1 if self.fused_relu else 0)
        if x._needs_grad() or (self.affine and (ga.requires_grad or be.requires_grad)):
            y.requires_grad = True

            def backward_fn(g: Tensor):
                dx = Tensor.empty(x.shape, x.dtype)
                dga = ga.grad_buffer() if self.affine else None
                dbe = be.grad_buffer() if self.affine else None
                lib.call(f"keydnn_cuda_bn2d_backward_bias_{s}", x.data, pb.data if pb is not None else None,
                         ga.data if ga else None, be.data if be else None, g.data, mean.data, invstd.data, dx.data,
                         dga.data if dga else None, dbe.data if dbe else None, N, C, H * W, 1 if self.fused_relu else 0)
                return (dx, dga, dbe) if self.affine else (dx,)

            y._ctx = Context((x, ga, be) if self.affine else (x,), backward_fn)
        follow = self.fused_pool or self.fused_gap      # shapes the fused kernels do not take: the layer itself
        return y if follow is None else follow(y)

    def _forward_averaged(self, x: Tensor, mean: Tensor, invstd: Tensor, ga, be, pb) -> Tensor:
        """BatchNorm (+ ReLU) and the GlobalAvgPool2d behind it in one pass each way: only the (N, C, 1, 1) means
        are written; backward spreads their gradient over the planes on the fly."""
        N, C, H, W = x.shape
        lib, s = x.native, _suffix(x.dtype)
        y = Tensor.empty((N, C, 1, 1), x.dtype)
        relu = 1 if self.fused_relu else 0
        lib.call(f"keydnn_cuda_bn2d_global_avgpool_forward_{s}", x.data, pb.data if pb is not None else None,
                 ga.data if ga else None, be.data if be else None, y.data, mean.data, invstd.data,
                 self.running_mean.data, self.running_var.data, N, C, H * W, _cfloat(x.dtype, self.eps),
                 _cfloat(x.dtype, self.momentum), 1 if self.training else 0, relu)
        if x._needs_grad() or (self.affine and (ga.requires_grad or be.requires_grad)):
            y.requires_grad = True

            def backward_fn(g: Tensor):
                dx = Tensor.empty(x.shape, x.dtype)
                dga = ga.grad_buffer() if self.affine else None
                dbe = be.grad_buffer() if self.affine else None
                lib.call(f"keydnn_cuda_bn2d_global_avgpool_backward_{s}", x.data, pb.data if pb is not None else None,
                         ga.data if ga else None, be.data if be else None, g.data, mean.data, invstd.data, dx.data,
                         dga.data if dga else None, dbe.data if dbe else None, N, C, H * W, relu)
                return (dx, dga, dbe) if self.affine else (dx,)

            y._ctx = Context((x, ga, be) if self.affine else (x,), backward_fn)
        return y

    def _forward_pooled(self, x: Tensor, mean: Tensor, invstd: Tensor, ga, be, pb) -> Tensor:
        """BatchNorm (+ ReLU) and the MaxPool2d(2) behind it in one pass each way: only the pooled tensor and its
        argmax positions are written; backward derives every element's gradient from them."""
        N, C, H, W = x.shape
        lib, s = x.native, _suffix(x.dtype)
        y = Tensor.empty((N, C, H // 2, W // 2), x.dtype)
        idx = CudaStorage.allocate(y.numel * 8, np.int64)
        relu = 1 if self.fused_relu else 0
        lib.call(f"keydnn_cuda_bn2d_maxpool2x2_forward_{s}", x.data, pb.data if pb is not None else None,
                 ga.data if ga else None, be.data if be else None, y.data, idx.dev_ptr, mean.data, invstd.data,
                 self.running_mean.data, self.running_var.data, N, C, H, W, _cfloat(x.dtype, self.eps),
                 _cfloat(x.dtype, self.momentum), 1 if self.training else 0, relu)
        if x._needs_grad() or (self.affine and (ga.requires_grad or be.requires_grad)):
            y.requires_grad = True

            def backward_fn(g: Tensor):
                dx = Tensor.empty(x.shape, x.dtype)
                dga = ga.grad_buffer() if self.affine else None
                dbe = be.grad_buffer() if self.affine else None
                lib.call(f"keydnn_cuda_bn2d_maxpool2x2_backward_{s}", x.data, pb.data if pb is not None else None,
                         ga.data if ga else None, be.data if be else None, g.data, idx.dev_ptr, mean.data, invstd.data,
                         dx.data, dga.data if dga else None, dbe.data if dbe else None, N, C, H, W, relu)
                return (dx, dga, dbe) if self.affine else (dx,)

            y._ctx = Context((x, ga, be) if self.affine else (x,), backward_fn)
        return y


class ReLU(Module):
    """``_activations.py:97-140`` over ``ReLUFn``: y = x * (x > 0), gradient g * (x > 0); one fused kernel each way."""

    def forward(self, x: Tensor) -> Tensor:
        from . import functional as F

        return F.relu(x)


class Flatten(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.reshape(x.shape[0], -1)


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=np.float32,
                 initializer: str = "kaiming") -> None:
        if initializer != "kaiming":
            raise ValueError("this mirror implements the 'kaiming' initializer (the benchmark's choice)")
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.weight = Parameter.from_numpy(kaiming_normal((out_features, in_features), np.dtype(dtype).type))
        self.bias = Parameter.from_numpy(np.zeros(out_features, dtype)) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        if x.ndim != 2 or x.shape[1] != self.in_features:
            raise ValueError(f"Linear expects (batch, {self.in_features}), got {x.shape}")
        dnn, lib, s = load_dnn(), x.native, _suffix(x.dtype)
        B, I, O = x.shape[0], self.in_features, self.out_features
        y = Tensor.empty((B, O), x.dtype)
        w, b = self.weight, self.bias
        dnn.call(f"keydnn_cuda_matmul_ex_{s}", x.data, w.data, y.data, B, O, I, 0, 1)          # x @ W.T
        if b is not None:
            lib.call(f"keydnn_cuda_bias_add_inplace_{s}", y.data, b.data, B, O)
        if x._needs_grad(w) or (b is not None and b.requires_grad):
            y.requires_grad = True

            def backward_fn(g: Tensor):
                gx = None
                if x.requires_grad:
                    gx = Tensor.empty(x.shape, x.dtype)
                    dnn.call(f"keydnn_cuda_matmul_ex_{s}", g.data, w.data, gx.data, B, I, O, 0, 0)      # g @ W
                gw = w.grad_buffer()
                dnn.call(f"keydnn_cuda_matmul_ex_{s}", g.data, x.data, gw.data, O, I, B, 1, 0)          # g.T @ x
                if b is None:
                    return (gx, gw)
                with no_grad():
                    gb = g.sum(axis=0)
                return (gx, gw, gb)

            y._ctx = Context((x, w) if b is None else (x, w, b), backward_fn)
        return y


class Sequential(Module):
    """Runs its layers in order (``models/_sequential.py:130-152``).  With ``fuse=True`` (default) a ReLU that
    directly follows a BatchNorm2d is folded into that layer's kernels, and the bias of a Conv2d that directly
    precedes a BatchNorm2d is added by the BatchNorm kernels as they read the activation (the convolution then
    skips its bias pass), and a MaxPool2d(2) or GlobalAvgPool2d that follows a BatchNorm2d (+ ReLU) is computed by
    the BatchNorm kernels as well (the normalised activation and its gradient are never stored).  Results are bit-identical to
    the separate layers."""

    def __init__(self, *layers, fuse: bool = True) -> None:
        self.layers = list(layers)
        self._skip = set()
        if fuse:
            for i in range(len(self.layers) - 1):
                a, b = self.layers[i], self.layers[i + 1]
                if isinstance(a, BatchNorm2d) and isinstance(b, ReLU) and a.gamma is not None:
                    a.fused_relu = True
                    self._skip.add(i + 1)
                if isinstance(a, Conv2d) and isinstance(b, BatchNorm2d) and a.bias is not None and a.bias.dtype == b.running_mean.dtype:
                    a.bias_deferred = True
                    b.pre_bias = a.bias
            for i, a in enumerate(self.layers):
                j = i + 1
                while j in self._skip:
                    j += 1
                nxt = self.layers[j] if j < len(self.layers) else None
                if (isinstance(a, BatchNorm2d) and isinstance(nxt, MaxPool2d) and nxt.kernel_size == (2, 2)
                        and nxt.stride == (2, 2) and nxt.padding == (0, 0)):
                    a.fused_pool = nxt         # pooled by the BatchNorm kernels; shapes they do not take go through nxt
                    self._skip.add(j)
                elif isinstance(a, BatchNorm2d) and isinstance(nxt, GlobalAvgPool2d):
                    a.fused_gap = nxt
                    self._skip.add(j)

    def forward(self, x: Tensor) -> Tensor:
        for i, layer in enumerate(self.layers):
            if i not in self._skip:
                x = layer(x)
        return x


def mse_loss(pred: Tensor, target: Tensor) -> Tensor:
    """``_losses.py:130-216``: mean((pred - target)^2) with the fused kernels of ``functional.MSEFn``; the backward takes
    the upstream scalar from the device, so a training step never waits for the host."""
    from . import functional as F

    return F.mse_loss(pred, target)


class _ViewStorage:
    """A window into a larger allocation; keeps the owner alive, frees nothing itself."""

    __slots__ = ("native", "device_index", "dev_ptr", "nbytes", "dtype", "_owner")

    def __init__(self, owner: CudaStorage, offset: int, nbytes: int, dtype) -> None:
        self.native, self.device_index = owner.native, owner.device_index
        self.dev_ptr, self.nbytes, self.dtype, self._owner = owner.dev_ptr + offset, nbytes, np.dtype(dtype), owner

    def incref(self) -> None:
        pass

    def decref(self) -> None:
        pass


class _FlatOptimizer:
    """Parameters, gradients and optimizer state in flat device buffers.

    All parameters are moved into one allocation (each at a 256-byte boundary; the ``Parameter`` objects
    become windows into it), so a step is: gather the gradients into a flat buffer, one in-place NCCL
    all-reduce over it when ``group.world > 1`` (its 1/world average is folded into the update kernel),
    one fused update kernel over the whole buffer.
    """

    graph_safe = True          # the launches of a step depend on nothing the host changes between steps

    def __init__(self, params: Iterable[Parameter], n_state: int, group=None) -> None:
        self.params = [p for p in params]
        if not self.params:
            raise ValueError(f"{type(self).__name__} needs at least one parameter")
        self.group = group
        self.dtype = self.params[0].dtype
        if any(p.dtype != self.dtype for p in self.params):
            raise TypeError("all parameters must share one dtype")
        isz = self.dtype.itemsize
        self.offsets: List[int] = []
        off = 0
        for p in self.params:
            self.offsets.append(off)
            off += (p.nbytes + 255) // 256 * 256
        self.n = off // isz
        self.native = self.params[0].native
        self.flat_p = CudaStorage.allocate(off, self.dtype)
        self.flat_g = CudaStorage.allocate(off, self.dtype)
        self.state = [CudaStorage.allocate(off, self.dtype) for _ in range(n_state)]
        for st in (self.flat_p, self.flat_g, *self.state):
            self.native.call("keydnn_cuda_memset", st.dev_ptr, 0, off)
        for p, o in zip(self.params, self.offsets):
            self.native.call("keydnn_cuda_memcpy_d2d", self.flat_p.dev_ptr + o, p.data, p.nbytes)
            p.storage = _ViewStorage(self.flat_p, o, p.nbytes, self.dtype)
            # gradients are written straight into the flat buffer by the layers that compute them
            p._grad_slot = Tensor(_ViewStorage(self.flat_g, o, p.nbytes, self.dtype), p.shape, self.dtype)
            p._slot_taken = False

    def zero_grad(self) -> None:
        for p in self.params:
            p.zero_grad()

    def _gather_grads(self) -> int:
        """Copies every gradient into the flat buffer, sums it over the ranks; returns the world size."""
        lib = self.native
        for p, o in zip(self.params, self.offsets):
            if p.grad is None:
                lib.call("keydnn_cuda_memset", self.flat_g.dev_ptr + o, 0, p.nbytes)
            elif p.grad.data != self.flat_g.dev_ptr + o:           # not already written in place (`Parameter.grad_buffer`)
                lib.call("keydnn_cuda_memcpy_d2d", self.flat_g.dev_ptr + o, p.grad.data, p.nbytes)
        world = 1 if self.group is None else self.group.world
        if world > 1:
            self.group.allreduce_sum(self.flat_g.dev_ptr, self.n, _suffix(self.dtype))
        return world

    def _segments(self):
        """(element offset, element count) pieces to update: the whole buffer when every parameter has a gradient;
        otherwise one piece per parameter that has one - a parameter without a gradient is skipped entirely, weight
        decay and state included, as the reference optimizers do (``optimizers/_sgd.py:127-129``, ``_adam.py:172-175``).
        With a process group every rank must see the same parameters without gradients."""
        if all(p.grad is not None for p in self.params):
            return [(0, self.n)]
        isz = self.dtype.itemsize
        return [(o // isz, p.numel) for p, o in zip(self.params, self.offsets) if p.grad is not None]


class SGD(_FlatOptimizer):
    """Stochastic gradient descent with coupled L2 weight decay (``optimizers/_sgd.py:119-140``) and
    optional momentum (an addition: v = momentum * v + g'; p -= lr * v), over flat buffers: one fused
    kernel over (p, g, v) where the reference runs five tensor passes and four allocations per parameter.
    """

    def __init__(self, params: Iterable[Parameter], lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0,
                 group=None) -> None:
        if lr <= 0.0:
            raise ValueError(f"lr must be > 0, got {lr}")
        if weight_decay < 0.0:
            raise ValueError(f"weight_decay must be >= 0, got {weight_decay}")
        super().__init__(params, 1 if momentum != 0.0 else 0, group)
        self.lr, self.momentum, self.weight_decay = float(lr), float(momentum), float(weight_decay)
        self.flat_v = self.state[0] if self.state else None

    def step(self) -> None:
        world = self._gather_grads()
        isz = self.dtype.itemsize
        for off, count in self._segments():
            self.native.call(f"keydnn_cuda_sgd_momentum_step_{_suffix(self.dtype)}", self.flat_p.dev_ptr + off * isz,
                             self.flat_g.dev_ptr + off * isz, self.flat_v.dev_ptr + off * isz if self.flat_v else None, count,
                             _cfloat(self.dtype, self.lr), _cfloat(self.dtype, self.momentum),
                             _cfloat(self.dtype, self.weight_decay), _cfloat(self.dtype, 1.0 / world))


class Adam(_FlatOptimizer):
    """Adam with coupled L2 weight decay (``optimizers/_adam.py:120-219``; there CPU-only, eleven tensor passes
    per parameter) over flat buffers: one fused kernel over (p, g, m, v) per step, the gradient all-reduce of
    ``group`` in front of it.  Every parameter shares the step count, as all of them get a gradient each step.
    The bias corrections 1 - beta^t change every step.  By default they are passed by value, so a step cannot be
    replayed from a CUDA graph (``graph_safe`` is False).  With ``device_step=True`` the step count lives on the
    device and the corrections come from a table built here in Python doubles (one entry per step until both are
    exactly 1 in the element type, a few ten thousand entries for the usual betas): same bits, and the step can
    be recorded."""

    graph_safe = False
    _MAX_TABLE = 1 << 21

    def __init__(self, params: Iterable[Parameter], lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, group=None, device_step: bool = False) -> None:
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(weight_decay)
        b1, b2 = self.betas
        if self.lr <= 0.0:
            raise ValueError(f"lr must be > 0, got {self.lr}")
        if not (0.0 < b1 < 1.0) or not (0.0 < b2 < 1.0):
            raise ValueError(f"betas must be in (0,1), got {self.betas}")
        if self.eps <= 0.0:
            raise ValueError(f"eps must be > 0, got {self.eps}")
        if self.weight_decay < 0.0:
            raise ValueError(f"weight_decay must be >= 0, got {self.weight_decay}")
        super().__init__(params, 2, group)
        self.flat_m, self.flat_v = self.state
        self.t = 0
        self._table = None
        if device_step:
            t_ = self.dtype.type
            rows, k = [], 1
            while True:
                a, b = t_(1.0 - b1 ** k), t_(1.0 - b2 ** k)
                rows.append((a, b))
                if a == 1 and b == 1:
                    break
                if len(rows) >= self._MAX_TABLE:
                    raise ValueError("betas too close to 1 for device_step: the correction table would not end")
                k += 1
            self._table = Tensor.from_numpy(np.asarray(rows, self.dtype))
            self._table_len = len(rows)
            self._count = CudaStorage.allocate(8, np.int64)
            self.native.call("keydnn_cuda_memset", self._count.dev_ptr, 0, 8)
            self._bias_now = Tensor.zeros((2,), self.dtype)
            self.graph_safe = True

    def step(self) -> None:
        world = self._gather_grads()
        self.t += 1
        b1, b2 = self.betas
        c = lambda v: _cfloat(self.dtype, v)   # noqa: E731
        if self._table is not None:
            if any(p.grad is None for p in self.params):
                raise RuntimeError("Adam(device_step=True) shares one device-side step count: every parameter needs a gradient")
            self.native.call(f"keydnn_cuda_adam_step_counted_{_suffix(self.dtype)}", self.flat_p.dev_ptr, self.flat_g.dev_ptr,
                             self.flat_m.dev_ptr, self.flat_v.dev_ptr, self.n, c(self.lr), c(b1), c(b2), c(self.eps),
                             c(self.weight_decay), c(1.0 - b1), c(1.0 - b2), self._table.data, self._table_len,
                             self._count.dev_ptr, self._bias_now.data, c(1.0 / world))
            return
        isz = self.dtype.itemsize
        for off, count in self._segments():
            b = off * isz
            self.native.call(f"keydnn_cuda_adam_step_{_suffix(self.dtype)}", self.flat_p.dev_ptr + b, self.flat_g.dev_ptr + b,
                             self.flat_m.dev_ptr + b, self.flat_v.dev_ptr + b, count, c(self.lr), c(b1), c(b2), c(self.eps),
                             c(self.weight_decay), c(1.0 - b1), c(1.0 - b2), c(1.0 - b1 ** self.t), c(1.0 - b2 ** self.t),
                             c(1.0 / world))


def small_cnn(dtype=np.float32) -> Sequential:
    """Conv(3->32,3x3,p1)-BN-ReLU-MaxPool(2)-Conv(32->64,3x3,p1)-BN-ReLU-GlobalAvgPool-Flatten-Linear(64->10)."""
    return Sequential(
        Conv2d(3, 32, 3, padding=1, dtype=dtype), BatchNorm2d(32, dtype=dtype), ReLU(), MaxPool2d(2),
        Conv2d(32, 64, 3, padding=1, dtype=dtype), BatchNorm2d(64, dtype=dtype), ReLU(), GlobalAvgPool2d(), Flatten(),
        Linear(64, 10, dtype=dtype),
    )


def train_step(model: Module, opt: SGD, x: Tensor, target: Tensor) -> Tensor:
    """zero_grad -> forward -> MSE -> backward -> optimizer step (``models/_models.py:402-513``); returns the loss tensor."""
    opt.zero_grad()
    loss = mse_loss(model(x), target)
    loss.backward()
    opt.step()
    return loss


class GraphedTrainStep:
    """``train_step`` recorded once into a CUDA graph and replayed with a single launch.

    The step is a fixed sequence of about a hundred kernel launches, library calls and small copies
    on buffers whose addresses repeat every step (the allocator hands the same blocks out in the
    same order), so after a few eager warm-up steps on a private stream it is captured; a replay
    costs one launch instead of ~1 ms of host-side enqueueing.  ``x`` and ``target`` are the fixed
    input buffers: copy each batch into them before ``run()``.  ``loss`` is the tensor the recorded
    step writes its loss to.  The reference has no counterpart (one host round trip per op).
    """

    def __init__(self, model: Module, opt: SGD, x: Tensor, target: Tensor, warmup: int = 3) -> None:
        if not getattr(opt, "graph_safe", False):
            raise TypeError(f"{type(opt).__name__} passes per-step values from the host; its step cannot be recorded")
        self.lib, self.dnn = x.native, load_dnn()
        self._keep = (model, opt, x, target)
        self._prev = ctypes.c_uint64(0)
        self.lib.call("keydnn_cuda_get_stream", ctypes.byref(self._prev))
        self.stream = ctypes.c_uint64(0)
        self.lib.call("keydnn_cuda_stream_create", ctypes.byref(self.stream))
        self.lib.call("keydnn_cuda_synchronize")
        self._use(self.stream.value)
        self.exec = ctypes.c_uint64(0)
        try:
            for _ in range(max(1, warmup)):
                self.loss = train_step(model, opt, x, target)
            self.lib.call("keydnn_cuda_stream_synchronize")
            self.lib.call("keydnn_cuda_graph_capture_begin")
            try:
                self.loss = train_step(model, opt, x, target)
            finally:
                self.lib.call("keydnn_cuda_graph_capture_end", ctypes.byref(self.exec))
        except Exception:
            self._use(self._prev.value)
            raise

    def _use(self, stream: int) -> None:
        # the cuDNN / cuBLAS library follows the operator library's stream (bound at load, `_native.load_dnn`)
        self.lib.call("keydnn_cuda_set_stream", stream)

    def run(self) -> Tensor:
        self.lib.call("keydnn_cuda_graph_launch", self.exec.value)
        return self.loss

    # -- pipelined feeding: batch i+1 crosses PCIe while step i runs ---------------------------------
    def _pipeline(self):
        if getattr(self, "_pipe", None) is None:
            lib = self.lib
            _, _, x, t = self._keep
            copy = ctypes.c_uint64(0)
            lib.call("keydnn_cuda_stream_create", ctypes.byref(copy))
            slots = []
            for _ in range(2):
                ev_in, ev_done, host = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_void_p(0)
                lib.call("keydnn_cuda_event_create", ctypes.byref(ev_in))
                lib.call("keydnn_cuda_event_create", ctypes.byref(ev_done))
                lib.call("keydnn_cuda_host_alloc", ctypes.byref(host), 16)
                slots.append({"x": Tensor.empty(x.shape, x.dtype), "t": Tensor.empty(t.shape, t.dtype), "arrived": ev_in.value,
                              "done": ev_done.value, "host": host.value,
                              "loss": np.frombuffer((ctypes.c_char * 16).from_address(host.value), dtype=self.loss.dtype, count=1)})
            self._pipe = {"copy": copy.value, "slots": slots, "n": 0}
        return self._pipe

    def step_async(self, host_x: np.ndarray, host_target: np.ndarray) -> int:
        """Enqueue one step on a batch in (pinned) host memory and return a ticket for ``loss_of``.

        The batch goes to one of two staging buffers on a copy stream, so it overlaps the step that is
        still running; the training stream then waits for it, moves it into the recorded step's input
        buffers (a device copy, microseconds), replays the step and copies its loss to pinned host memory.
        Nothing here waits for the GPU."""
        lib, pipe = self.lib, self._pipeline()
        _, _, x, t = self._keep
        k = pipe["n"] % 2
        slot = pipe["slots"][k]
        pipe["n"] += 1
        lib.call("keydnn_cuda_set_stream", pipe["copy"])
        lib.call("keydnn_cuda_stream_wait_event", slot["done"])          # the step that last read this slot is over
        lib.call("keydnn_cuda_memcpy_h2d_async", slot["x"].data, host_x.ctypes.data, host_x.nbytes)
        lib.call("keydnn_cuda_memcpy_h2d_async", slot["t"].data, host_target.ctypes.data, host_target.nbytes)
        lib.call("keydnn_cuda_event_record", slot["arrived"])
        lib.call("keydnn_cuda_set_stream", self.stream.value)
        lib.call("keydnn_cuda_stream_wait_event", slot["arrived"])
        lib.call("keydnn_cuda_memcpy_d2d", x.data, slot["x"].data, x.nbytes)
        lib.call("keydnn_cuda_memcpy_d2d", t.data, slot["t"].data, t.nbytes)
        lib.call("keydnn_cuda_graph_launch", self.exec.value)
        lib.call("keydnn_cuda_memcpy_d2h_async", slot["host"], self.loss.data, self.loss.nbytes)
        lib.call("keydnn_cuda_event_record", slot["done"])
        return k

    def loss_of(self, ticket: int) -> float:
        """The loss of the step ``step_async`` returned ``ticket`` for (waits for that step only)."""
        slot = self._pipe["slots"][ticket]
        self.lib.call("keydnn_cuda_event_synchronize", slot["done"])
        return float(slot["loss"][0])

    def close(self) -> None:
        pipe = getattr(self, "_pipe", None)
        if pipe is not None:
            self.lib.call("keydnn_cuda_synchronize")
            for slot in pipe["slots"]:
                self.lib.call("keydnn_cuda_event_destroy", slot["arrived"])
                self.lib.call("keydnn_cuda_event_destroy", slot["done"])
                self.lib.call("keydnn_cuda_host_free", slot["host"])
            self.lib.call("keydnn_cuda_stream_destroy", pipe["copy"])
            self._pipe = None
        if self.exec.value:
            self.lib.call("keydnn_cuda_graph_destroy", self.exec.value)
            self.exec = ctypes.c_uint64(0)
        self.lib.call("keydnn_cuda_stream_synchronize")
        self._use(self._prev.value)
