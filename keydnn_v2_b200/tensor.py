"""CUDA Tensor with reverse-mode autograd, driving ``libkeydnn_b200.so``.

Host-side mirror of the part of the reference's Tensor that sits on the CUDA hot
path: the CUDA control paths of ``src/keydnn/infrastructure/tensor/mixins/``
(arithmetic, comparison, reduction, memory) with their backward closures, the
``Context`` of ``tensor/_tensor_context.py:8-56`` and the CUDA branch of
``Tensor.backward`` (``tensor/_tensor.py:1601-1861``).  Same names, argument
meaning and error behaviour for that path; nothing here computes on the CPU, and
a missing native library raises at the first allocation.

Differences from the reference that are visible only as speed:
  * outputs come from the library's caching pool (no ``cudaMalloc``/``cudaFree`` per op);
  * ops enqueue and return; the host waits only in ``to_numpy`` / ``item`` /
    ``synchronize`` (the reference synchronises after most reductions and pools);
  * ``max`` backward writes the whole gradient in one kernel (no zero-fill pass).
"""
from __future__ import annotations

import ctypes
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from ._cuda_storage import CudaStorage
from ._native import Native

Number = Union[int, float]
_INT32_MAX = 2**31 - 1


def _suffix(dtype) -> str:
    dt = np.dtype(dtype)
    if dt == np.float32:
        return "f32"
    if dt == np.float64:
        return "f64"
    raise TypeError(f"CUDA ops support float32/float64 only, got {dt}")


def _numel(shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class Device:
    """``Device("cuda:0")``; the CUDA control paths of the reference are registered for that
    device only (``domain/device/_device.py:124-155``), one process per GPU."""

    def __init__(self, spec: str = "cuda:0") -> None:
        kind, _, idx = str(spec).partition(":")
        if kind != "cuda":
            raise ValueError("this package implements the CUDA path only; use Device('cuda:0')")
        self.type = "cuda"
        self.index = int(idx or 0)

    def is_cuda(self) -> bool:
        return True

    def is_cpu(self) -> bool:
        return False

    def __eq__(self, other) -> bool:
        return isinstance(other, Device) and other.index == self.index

    def __hash__(self) -> int:
        return hash(("cuda", self.index))

    def __repr__(self) -> str:
        return f"Device('cuda:{self.index}')"


class Context:
    """Backward record of one op (``tensor/_tensor_context.py:8-56``)."""

    __slots__ = ("parents", "backward_fn", "saved_tensors", "saved_meta")

    def __init__(self, parents: Sequence["Tensor"], backward_fn: Callable[["Tensor"], Sequence[Optional["Tensor"]]]):
        self.parents = tuple(parents)
        self.backward_fn = backward_fn
        self.saved_tensors: List["Tensor"] = []
        self.saved_meta: Dict[str, object] = {}

    def save_for_backward(self, *tensors: "Tensor") -> None:
        self.saved_tensors.extend(tensors)


_GRAD_ENABLED = True


class no_grad:
    def __enter__(self):
        global _GRAD_ENABLED
        self._prev = _GRAD_ENABLED
        _GRAD_ENABLED = False

    def __exit__(self, *exc):
        global _GRAD_ENABLED
        _GRAD_ENABLED = self._prev


class Tensor:
    __slots__ = ("storage", "shape", "dtype", "device", "requires_grad", "grad", "_ctx", "native", "_is_unit_seed",
                 "__weakref__")

    # ------------------------------------------------------------------ build
    def __init__(self, storage: CudaStorage, shape: Sequence[int], dtype, *, device: Optional[Device] = None,
                 requires_grad: bool = False, ctx: Optional[Context] = None) -> None:
        self.storage = storage
        self.shape = tuple(int(d) for d in shape)
        self.dtype = np.dtype(dtype)
        self.device = device or Device("cuda:0")
        self.requires_grad = bool(requires_grad)
        self.grad: Optional[Tensor] = None
        self._ctx = ctx
        self._is_unit_seed = False      # True for the implicit gradient of ones that backward() seeds
        self.native: Native = storage.native

    @classmethod
    def _from_storage(cls, storage, *, shape, dtype, device=None, requires_grad=False) -> "Tensor":
        return cls(storage, shape, dtype, device=device, requires_grad=requires_grad)

    @classmethod
    def empty(cls, shape: Sequence[int], dtype=np.float32, *, requires_grad: bool = False) -> "Tensor":
        dt = np.dtype(dtype)
        st = CudaStorage.allocate(_numel(shape) * dt.itemsize, dt)
        return cls(st, shape, dt, requires_grad=requires_grad)

    @classmethod
    def full(cls, shape: Sequence[int], value: Number, dtype=np.float32, *, requires_grad: bool = False) -> "Tensor":
        t = cls.empty(shape, dtype, requires_grad=requires_grad)
        t.fill_(value)
        return t

    @classmethod
    def zeros(cls, shape, dtype=np.float32, *, requires_grad: bool = False) -> "Tensor":
        return cls.full(shape, 0.0, dtype, requires_grad=requires_grad)

    @classmethod
    def ones(cls, shape, dtype=np.float32, *, requires_grad: bool = False) -> "Tensor":
        return cls.full(shape, 1.0, dtype, requires_grad=requires_grad)

    @classmethod
    def from_numpy(cls, arr: np.ndarray, *, requires_grad: bool = False) -> "Tensor":
        a = np.ascontiguousarray(arr)
        if a.dtype not in (np.float32, np.float64, np.int64):
            a = a.astype(np.float32)
        t = cls.empty(a.shape, a.dtype, requires_grad=requires_grad) if a.dtype != np.int64 else cls(
            CudaStorage.allocate(a.nbytes, a.dtype), a.shape, a.dtype)
        t.copy_from_numpy(a)
        return t

    # ------------------------------------------------------------- basic info
    @property
    def data(self) -> int:
        """Device pointer as an integer (what crosses the C ABI)."""
        return self.storage.dev_ptr

    @property
    def numel(self) -> int:
        return _numel(self.shape)

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def nbytes(self) -> int:
        return self.numel * self.dtype.itemsize

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, device={self.device}, requires_grad={self.requires_grad})"

    # ------------------------------------------------------------ host copies
    def copy_from_numpy(self, arr: np.ndarray) -> None:
        a = np.ascontiguousarray(arr, dtype=self.dtype)
        if a.shape != self.shape:
            raise ValueError(f"shape mismatch: tensor {self.shape} vs array {a.shape}")
        if a.nbytes:
            self.native.call("keydnn_cuda_memcpy_h2d", self.data, a.ctypes.data, a.nbytes)

    def to_numpy(self, out: Optional[np.ndarray] = None) -> np.ndarray:
        if out is None:
            out = np.empty(self.shape, self.dtype)
        if out.nbytes:
            self.native.call("keydnn_cuda_memcpy_d2h", out.ctypes.data, self.data, out.nbytes)
        return out

    def item(self) -> float:
        if self.numel != 1:
            raise ValueError("item() needs a one-element tensor")
        return float(self.to_numpy().reshape(-1)[0])

    def synchronize(self) -> None:
        self.native.call("keydnn_cuda_synchronize")

    def copy_from(self, other: "Tensor") -> None:
        """Device-to-device copy (``tensor/mixins/memory/_base.py`` copy_from)."""
        if other.shape != self.shape or other.dtype != self.dtype:
            raise ValueError("copy_from needs equal shape and dtype")
        self.native.call("keydnn_cuda_memcpy_d2d", self.data, other.data, self.nbytes)

    def clone(self) -> "Tensor":
        out = Tensor.empty(self.shape, self.dtype)
        out.copy_from(self)
        return out

    def detach(self) -> "Tensor":
        self.storage.incref()
        return Tensor(self.storage, self.shape, self.dtype, device=self.device)

    def fill_(self, value: Number) -> "Tensor":
        if self.numel:
            arg = ctypes.c_float(value) if self.dtype == np.float32 else ctypes.c_double(value)
            self.native.call(f"keydnn_cuda_fill_{_suffix(self.dtype)}", self.data, self.numel, arg)
        return self

    def zero_grad(self) -> None:
        self.grad = None

    # -------------------------------------------------------------- internals
    def _new_like(self, shape=None, dtype=None) -> "Tensor":
        return Tensor.empty(self.shape if shape is None else shape, self.dtype if dtype is None else dtype)

    def _needs_grad(self, *others: "Tensor") -> bool:
        return _GRAD_ENABLED and (self.requires_grad or any(o.requires_grad for o in others))

    def _check_same(self, other: "Tensor", op: str) -> None:
        if not isinstance(other, Tensor):
            raise TypeError(f"{op}: expected a Tensor, got {type(other).__name__}")
        if other.shape != self.shape:
            raise ValueError(f"{op}: shape mismatch {self.shape} vs {other.shape}")
        if other.dtype != self.dtype:
            raise TypeError(f"{op}: dtype mismatch {self.dtype} vs {other.dtype}")

    def _binary(self, name: str, other: "Tensor", out_dtype=None) -> "Tensor":
        self._check_same(other, name)
        out = self._new_like(dtype=out_dtype)
        n = self.numel
        if n:
            suf = _suffix(self.dtype)
            if name == "mul":
                fn = f"keydnn_cuda_mul_{suf}" if n <= _INT32_MAX else f"keydnn_cuda_mul64_{suf}"
            else:
                fn = f"keydnn_cuda_{name}_{suf}"
            self.native.call(fn, self.data, other.data, out.data, n)
        return out

    def _scalar(self, name: str, alpha: Number, out_dtype=None) -> "Tensor":
        out = self._new_like(dtype=out_dtype)
        n = self.numel
        if n:
            suf = _suffix(self.dtype)
            arg = ctypes.c_float(alpha) if self.dtype == np.float32 else ctypes.c_double(alpha)
            if name == "mul_scalar" and n > _INT32_MAX:
                raise ValueError("mul_scalar supports at most 2^31-1 elements (reference ABI: int numel)")
            self.native.call(f"keydnn_cuda_{name}_{suf}", self.data, arg, out.data, n)
        return out

    @staticmethod
    def _muldiv_backward(kind: str, g: "Tensor", a: "Tensor", b: "Tensor"):
        ga = Tensor.empty(a.shape, a.dtype) if a.requires_grad else None
        gb = Tensor.empty(b.shape, b.dtype) if b.requires_grad else None
        if a.numel and (ga is not None or gb is not None):
            a.native.call(f"keydnn_cuda_{kind}_backward_{_suffix(a.dtype)}", g.data, a.data, b.data,
                          ga.data if ga is not None else None, gb.data if gb is not None else None, a.numel)
        return (ga, gb)

    def _as_tensor_like(self, value: Number) -> "Tensor":
        """Scalar lifted to a filled tensor (``tensor/_tensor.py:722-754``)."""
        return Tensor.full(self.shape, value, self.dtype)

    # ------------------------------------------------------------- arithmetic
    def __add__(self, other):
        if isinstance(other, Tensor):
            out = self._binary("add", other)
            if self._needs_grad(other):
                out.requires_grad = True
                # both parents receive grad_out itself (_tensor_addition.py:102-107)
                out._ctx = Context((self, other), lambda g: (g, g))
            return out
        out = self._scalar("add_scalar", other)
        if self._needs_grad():
            out.requires_grad = True
            out._ctx = Context((self,), lambda g: (g,))
        return out

    __radd__ = __add__

    def __sub__(self, other):
        if isinstance(other, Tensor):
            out = self._binary("sub", other)
            if self._needs_grad(other):
                out.requires_grad = True
                out._ctx = Context((self, other), lambda g: (g, -g))   # _tensor_subtraction.py:97
            return out
        out = self._scalar("sub_scalar", other)
        if self._needs_grad():
            out.requires_grad = True
            out._ctx = Context((self,), lambda g: (g,))
        return out

    def __rsub__(self, other):
        # scalar - tensor: the scalar is lifted to a tensor (arithmetic/_base.py:204-205)
        return self._as_tensor_like(other) - self

    def __mul__(self, other):
        if isinstance(other, Tensor):
            out = self._binary("mul", other)
            if self._needs_grad(other):
                out.requires_grad = True
                a, b = self, other

                def backward_fn(g: "Tensor"):
                    # (g*b, g*a) as in _tensor_multiplication.py:98-103, both in one pass over g, a, b
                    return a._muldiv_backward("mul", g, a, b)

                out._ctx = Context((a, b), backward_fn)
            return out
        out = self._scalar("mul_scalar", other)
        if self._needs_grad():
            out.requires_grad = True
            alpha = other

            def backward_fn(g: "Tensor"):
                with no_grad():
                    return (g * alpha,)

            out._ctx = Context((self,), backward_fn)
        return out

    __rmul__ = __mul__

    def __truediv__(self, other):
        if isinstance(other, Tensor):
            out = self._binary("div", other)
            if self._needs_grad(other):
                out.requires_grad = True
                a, b = self, other

                def backward_fn(g: "Tensor"):
                    # (g/b, -(g*a)/(b*b)) as in _tensor_division.py:104-114, both in one pass
                    return a._muldiv_backward("div", g, a, b)

                out._ctx = Context((a, b), backward_fn)
            return out
        out = self._scalar("div_scalar", other)
        if self._needs_grad():
            out.requires_grad = True
            alpha = other

            def backward_fn(g: "Tensor"):
                with no_grad():
                    return (g / alpha,)

            out._ctx = Context((self,), backward_fn)
        return out

    def __rtruediv__(self, other):
        return self._as_tensor_like(other) / self     # arithmetic/_base.py:86-87

    def __neg__(self):
        out = self._new_like()
        if self.numel:
            self.native.call(f"keydnn_cuda_neg_{_suffix(self.dtype)}", self.data, out.data, self.numel)
        if self._needs_grad():
            out.requires_grad = True
            out._ctx = Context((self,), lambda g: (-g,))
        return out

    # in-place forms: reached only for tensors outside the graph, as in the
    # reference (arithmetic/_base.py:207-615: requires_grad or a ctx forces the
    # out-of-place fallback `out = a op b; a.copy_from(out)`).
    def _inplace(self, name: str, other) -> "Tensor":
        safe = not self.requires_grad and self._ctx is None
        suf = _suffix(self.dtype)
        n = self.numel
        if isinstance(other, Tensor):
            self._check_same(other, name)
            if not safe:
                with no_grad():
                    tmp = self._binary(name, other)
                self.copy_from(tmp)
                return self
            if n:
                if name == "mul" and n > _INT32_MAX:
                    raise ValueError("mul_inplace supports at most 2^31-1 elements")
                self.native.call(f"keydnn_cuda_{name}_inplace_{suf}", self.data, other.data, n)
            return self
        if not safe:
            with no_grad():
                tmp = self._scalar(f"{name}_scalar", other)
            self.copy_from(tmp)
            return self
        if n:
            arg = ctypes.c_float(other) if self.dtype == np.float32 else ctypes.c_double(other)
            self.native.call(f"keydnn_cuda_{name}_scalar_inplace_{suf}", self.data, arg, n)
        return self

    def __iadd__(self, other):
        return self._inplace("add", other)

    def __isub__(self, other):
        return self._inplace("sub", other)

    def __imul__(self, other):
        return self._inplace("mul", other)

    def __itruediv__(self, other):
        return self._inplace("div", other)

    # -------------------------------------------------------------- comparison
    def _compare(self, name: str, other) -> "Tensor":
        # float32 1.0/0.0 masks whatever the input type; no gradient (_tensor_gt.py:37-116)
        if isinstance(other, Tensor):
            return self._binary(name, other, out_dtype=np.float32)
        return self._scalar(f"{name}_scalar", other, out_dtype=np.float32)

    def __gt__(self, other):
        return self._compare("gt", other)

    def __ge__(self, other):
        return self._compare("ge", other)

    def __lt__(self, other):
        return self._compare("lt", other)

    def __le__(self, other):
        return self._compare("le", other)

    def eq(self, other):
        return self._compare("eq", other)

    def ne(self, other):
        return self._compare("ne", other)

    # ----------------------------------------------------------------- memory
    def reshape(self, *shape) -> "Tensor":
        """Alias of the same storage (``tensor/mixins/memory/_base.py:840-915``)."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = list(int(d) for d in shape)
        if shape.count(-1) == 1:
            known = _numel([d for d in shape if d != -1])
            shape[shape.index(-1)] = self.numel // max(known, 1)
        if _numel(shape) != self.numel:
            raise ValueError(f"cannot reshape {self.shape} to {tuple(shape)}")
        self.storage.incref()
        out = Tensor(self.storage, shape, self.dtype, device=self.device)
        if self._needs_grad():
            out.requires_grad = True
            src_shape = self.shape
            out._ctx = Context((self,), lambda g: (g.reshape(src_shape),))
        return out

    def broadcast_to(self, shape: Sequence[int]) -> "Tensor":
        shape = tuple(int(d) for d in shape)
        out = Tensor.empty(shape, self.dtype)
        ins = np.asarray(self.shape, dtype=np.int64)
        outs = np.asarray(shape, dtype=np.int64)
        self.native.call(f"keydnn_cuda_broadcast_to_{_suffix(self.dtype)}", self.data, out.data,
                         ins.ctypes.data if ins.size else outs.ctypes.data, len(self.shape), outs.ctypes.data, len(shape))
        if self._needs_grad():
            out.requires_grad = True
            src_shape = self.shape
            pad = (1,) * (len(shape) - len(src_shape)) + src_shape

            def backward_fn(g: "Tensor"):
                with no_grad():     # _tensor_broadcast.py:117-146
                    return (g.sum_to_shape(pad).reshape(src_shape),)

            out._ctx = Context((self,), backward_fn)
        return out

    def sum_to_shape(self, shape: Sequence[int]) -> "Tensor":
        shape = tuple(int(d) for d in shape)
        if len(shape) != self.ndim:
            raise ValueError("sum_to_shape needs a target of the same rank")
        out = Tensor.empty(shape, self.dtype)
        ins = np.asarray(self.shape, dtype=np.int64)
        outs = np.asarray(shape, dtype=np.int64)
        self.native.call(f"keydnn_cuda_sum_to_shape_{_suffix(self.dtype)}", self.data, out.data, ins.ctypes.data,
                         outs.ctypes.data, self.ndim)
        if self._needs_grad():
            out.requires_grad = True
            src_shape = self.shape

            def backward_fn(g: "Tensor"):
                with no_grad():     # _tensor_sum_to_shape.py:193-272
                    return (g.broadcast_to(src_shape),)

            out._ctx = Context((self,), backward_fn)
        return out

    # -------------------------------------------------------------- reductions
    def _matrix_dims(self, op: str) -> Tuple[int, int]:
        if self.ndim != 2:
            raise ValueError(f"{op}(axis=...) on CUDA needs a 2-D tensor, got shape {self.shape}")
        return self.shape

    def sum(self, axis: Optional[int] = None, keepdims: bool = False) -> "Tensor":
        suf = _suffix(self.dtype)
        if axis is None:
            out = Tensor.empty((), self.dtype)
            self.native.call(f"keydnn_cuda_sum_all_{suf}", self.data, out.data, self.numel)
            if self._needs_grad():
                out.requires_grad = True
                src = self

                def backward_fn(g: "Tensor"):
                    gx = Tensor.empty(src.shape, src.dtype)      # _tensor_sum.py:99-164
                    src.native.call(f"keydnn_cuda_sum_backward_fill_{suf}", g.data, gx.data, src.numel)
                    return (gx,)

                out._ctx = Context((self,), backward_fn)
            return out
        rows, cols = self._matrix_dims("sum")
        ax = axis if axis >= 0 else axis + 2
        if ax not in (0, 1):
            raise ValueError(f"axis {axis} out of bounds for ndim 2")
        n_out = cols if ax == 0 else rows
        kshape = ((1, cols) if ax == 0 else (rows, 1)) if keepdims else (n_out,)
        out = Tensor.empty(kshape, self.dtype)
        self.native.call(f"keydnn_cuda_sum_axis2d_forward_{suf}", self.data, out.data, rows, cols, ax)
        if self._needs_grad():
            out.requires_grad = True
            src = self

            def backward_fn(g: "Tensor"):
                gx = Tensor.empty(src.shape, src.dtype)          # _tensor_sum.py:191-316
                src.native.call(f"keydnn_cuda_sum_axis2d_backward_{suf}", g.data, gx.data, rows, cols, ax)
                return (gx,)

            out._ctx = Context((self,), backward_fn)
        return out

    def mean(self, axis: Optional[int] = None, keepdims: bool = False) -> "Tensor":
        """All-elements mean as in the reference (``_tensor_mean.py:91-192``); ``axis`` is an
        addition (the reference's ``mean`` takes none)."""
        suf = _suffix(self.dtype)
        if axis is None:
            out = Tensor.empty((), self.dtype)
            self.native.call(f"keydnn_cuda_mean_all_{suf}", self.data, out.data, self.numel)
            if self._needs_grad():
                out.requires_grad = True
                src = self

                def backward_fn(g: "Tensor"):
                    gx = Tensor.empty(src.shape, src.dtype)
                    src.native.call(f"keydnn_cuda_mean_backward_fill_{suf}", g.data, gx.data, src.numel)
                    return (gx,)

                out._ctx = Context((self,), backward_fn)
            return out
        rows, cols = self._matrix_dims("mean")
        ax = axis if axis >= 0 else axis + 2
        if ax not in (0, 1):
            raise ValueError(f"axis {axis} out of bounds for ndim 2")
        n_out = cols if ax == 0 else rows
        kshape = ((1, cols) if ax == 0 else (rows, 1)) if keepdims else (n_out,)
        out = Tensor.empty(kshape, self.dtype)
        self.native.call(f"keydnn_cuda_mean_axis2d_forward_{suf}", self.data, out.data, rows, cols, ax)
        if self._needs_grad():
            out.requires_grad = True
            src = self

            def backward_fn(g: "Tensor"):
                gx = Tensor.empty(src.shape, src.dtype)
                src.native.call(f"keydnn_cuda_mean_axis2d_backward_{suf}", g.data, gx.data, rows, cols, ax)
                return (gx,)

            out._ctx = Context((self,), backward_fn)
        return out

    def max(self, axis: Optional[int] = -1, keepdims: bool = False) -> "Tensor":
        """2-D, axis 0/1 as in the reference (``_tensor_max.py:22-169``): values plus an int64
        first-occurrence index kept for backward, which routes the gradient to that single
        position.  ``axis=None`` (all elements) is an addition."""
        suf = _suffix(self.dtype)
        if axis is None:
            out = Tensor.empty((), self.dtype)
            idx = CudaStorage.allocate(8, np.int64)
            self.native.call(f"keydnn_cuda_max_all_forward_{suf}", self.data, out.data, idx.dev_ptr, self.numel)
            if self._needs_grad():
                out.requires_grad = True
                src = self

                def backward_fn(g: "Tensor"):
                    gx = Tensor.empty(src.shape, src.dtype)
                    src.native.call(f"keydnn_cuda_max_all_backward_{suf}", g.data, idx.dev_ptr, gx.data, src.numel)
                    return (gx,)

                out._ctx = Context((self,), backward_fn)
                out._ctx.saved_meta["argmax_idx"] = idx
            return out
        rows, cols = self._matrix_dims("max")
        ax = axis if axis >= 0 else axis + 2
        if ax not in (0, 1):
            raise ValueError(f"axis {axis} out of bounds for ndim 2")
        n_out = cols if ax == 0 else rows
        kshape = ((1, cols) if ax == 0 else (rows, 1)) if keepdims else (n_out,)
        out = Tensor.empty(kshape, self.dtype)
        idx = CudaStorage.allocate(n_out * 8, np.int64)
        self.native.call(f"keydnn_cuda_max_axis2d_forward_{suf}", self.data, out.data, idx.dev_ptr, rows, cols, ax)
        if self._needs_grad():
            out.requires_grad = True
            src = self

            def backward_fn(g: "Tensor"):
                gx = Tensor.empty(src.shape, src.dtype)          # _tensor_max.py:152-162
                src.native.call(f"keydnn_cuda_max_axis2d_backward_ex_{suf}", g.data, idx.dev_ptr, gx.data, rows, cols, ax)
                return (gx,)

            out._ctx = Context((self,), backward_fn)
            out._ctx.saved_meta["argmax_idx"] = idx
            out._ctx.saved_meta["axis"] = ax
        return out

    # ---------------------------------------------------------------- autograd
    # ------------------------------------------------------------------ unary
    def exp(self) -> "Tensor":
        """``tensor/mixins/unary/_tensor_exp.py:40-80``."""
        from . import functional as F

        return F.exp(self)

    def log(self) -> "Tensor":
        """``tensor/mixins/unary/_tensor_log.py:60-123`` (on the device here)."""
        from . import functional as F

        return F.log(self)

    def sqrt(self) -> "Tensor":
        """``tensor/mixins/unary/_tensor_sqrt.py:60-125`` (on the device here)."""
        from . import functional as F

        return F.sqrt(self)

    def _set_ctx(self, ctx: Optional[Context]) -> None:
        self._ctx = ctx

    def backward(self, grad_out: Optional["Tensor"] = None, *, retain_graph: bool = False) -> None:
        """Reverse topological walk (``tensor/_tensor.py:1601-1861``): seed with ``grad_out``
        (ones for a scalar), call each ``ctx.backward_fn``, add contributions that meet at
        a tensor (the first two out of place, later ones in place into that private sum),
        store the result on leaves that require grad.  Unless ``retain_graph`` is
        set, every visited node drops its Context afterwards, which releases the saved
        activations to the allocator at once."""
        if not self.requires_grad:
            raise RuntimeError("backward() on a tensor that does not require grad")
        if grad_out is None:
            if self.numel != 1:
                raise ValueError("grad_out must be given for non-scalar tensors")
            grad_out = Tensor.full(self.shape, 1.0, self.dtype)
            grad_out._is_unit_seed = True
        elif grad_out.shape != self.shape:
            raise ValueError(f"grad_out shape {grad_out.shape} != tensor shape {self.shape}")

        topo: List[Tensor] = []
        seen = set()
        stack: List[Tuple[Tensor, bool]] = [(self, False)]
        while stack:
            node, done = stack.pop()
            if done:
                topo.append(node)
                continue
            if id(node) in seen:
                continue
            seen.add(id(node))
            stack.append((node, True))
            if node._ctx is not None:
                for p in node._ctx.parents:
                    if p.requires_grad and id(p) not in seen:
                        stack.append((p, False))

        grads: Dict[int, Tensor] = {id(self): grad_out}
        owned = set()       # ids of sums made here: nobody else sees them, so further terms are added in place
        with no_grad():
            for node in reversed(topo):
                g = grads.pop(id(node), None)
                if g is None:
                    continue
                if node._ctx is None:
                    node.grad = g if node.grad is None else node.grad + g
                    continue
                parent_grads = node._ctx.backward_fn(g)
                if len(parent_grads) != len(node._ctx.parents):
                    raise RuntimeError("backward_fn returned a wrong number of gradients")
                for p, pg in zip(node._ctx.parents, parent_grads):
                    if pg is None or not p.requires_grad:
                        continue
                    if pg.shape != p.shape:
                        raise RuntimeError(f"gradient shape {pg.shape} != parent shape {p.shape}")
                    prev = grads.get(id(p))
                    if prev is None:
                        grads[id(p)] = pg
                    elif id(prev) in owned:
                        prev += pg              # third and later terms: no new tensor (tensor/_tensor.py:2487 wishes for this)
                    else:
                        total = prev + pg       # first meeting: either term may be shared with another branch
                        owned.add(id(total))
                        grads[id(p)] = total
                if not retain_graph:
                    node._ctx = None


class Parameter(Tensor):
    """Trainable leaf (``src/keydnn/infrastructure/_parameter.py``).

    An optimizer that keeps all gradients in one flat buffer may give a parameter a *gradient slot*: a tensor
    of the parameter's shape inside that buffer.  The layer that computes the parameter's gradient asks for
    ``grad_buffer()`` instead of allocating one and so writes the gradient where the optimizer (and the
    gradient all-reduce in front of it) reads it: no copy per parameter and step.  The slot is handed out once
    per step (``zero_grad`` re-arms it); a parameter used twice in a graph gets an ordinary buffer the second
    time and the autograd walk adds the two as it always does."""

    __slots__ = ("_grad_slot", "_slot_taken")

    def __init__(self, storage, shape, dtype, **kw) -> None:
        kw["requires_grad"] = True
        super().__init__(storage, shape, dtype, **kw)
        self._grad_slot: Optional[Tensor] = None
        self._slot_taken = False

    def grad_buffer(self) -> Tensor:
        """Where the gradient of this parameter should be written by the kernel that computes it."""
        if self._grad_slot is not None and not self._slot_taken:
            self._slot_taken = True
            return self._grad_slot
        return Tensor.empty(self.shape, self.dtype)

    def zero_grad(self) -> None:
        self.grad = None
        self._slot_taken = False

    @classmethod
    def from_numpy(cls, arr: np.ndarray, **_) -> "Parameter":
        a = np.ascontiguousarray(arr)
        st = CudaStorage.allocate(a.nbytes, a.dtype)
        p = cls(st, a.shape, a.dtype)
        p.copy_from_numpy(a)
        return p
