"""Row-sharded reductions: each rank owns ``rows`` consecutive rows of a
(``rows * world``, ``cols``) matrix.

  axis=1           per-row results: local, no exchange.
  axis=0 / None    sum, mean: local partial -> in-place NCCL all-reduce of the (cols,) vector or
                   scalar on the same stream -> the 1/count scale of the mean is applied after it.
                   max: local (value, first row) pairs -> all-gather -> per-column selection
                   "greater value, else lower rank" (NCCL has no MAXLOC).
  backward         every rank writes its own rows of the gradient; for max only the rank that
                   owns the maximum writes the routed value.

With world == 1 the same calls run without any collective.  Buffers are allocated once; a call
enqueues kernels and returns.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import numpy as np

from ._cuda_storage import CudaStorage
from .distributed import Group, single
from .tensor import Tensor, _suffix


class ShardedReductions:
    def __init__(self, x: Tensor, group: Optional[Group] = None) -> None:
        if x.ndim != 2:
            raise ValueError("ShardedReductions needs a 2-D local shard")
        self.x = x
        self.g = group or single(x.native)
        self.lib = x.native
        self.rows, self.cols = x.shape
        self.dt = x.dtype
        self.suf = _suffix(self.dt)
        w = self.g.world
        n_max = max(self.rows, self.cols)
        isz = self.dt.itemsize
        self.out = Tensor.empty((n_max,), self.dt)             # reduction result
        self.idx = CudaStorage.allocate(n_max * 8, np.int64)   # local argmax
        self.idx_global = CudaStorage.allocate(self.cols * 8, np.int64)
        self.idx_local = CudaStorage.allocate(self.cols * 8, np.int64)
        self.gather_val = CudaStorage.allocate(max(w * self.cols * isz, 16), self.dt)
        self.gather_idx = CudaStorage.allocate(max(w * self.cols * 8, 16), np.int64)
        self.sel_val = Tensor.empty((self.cols,), self.dt)
        self.ones = Tensor.ones((n_max,), self.dt)             # upstream gradient
        self.go = Tensor.empty((n_max,), self.dt)
        self.gx = Tensor.empty(x.shape, self.dt)

    def _c(self, v: float):
        return ctypes.c_float(v) if self.dt == np.float32 else ctypes.c_double(v)

    # ------------------------------------------------------------------ forward
    def forward(self, op: str, axis: Optional[int]) -> Tuple[int, int]:
        """Runs one reduction; returns (device pointer, element count) of the result."""
        lib, x, s, g = self.lib, self.x, self.suf, self.g
        rows, cols, w = self.rows, self.cols, self.g.world
        out = self.out.data
        if op in ("sum", "mean"):
            if axis == 1:
                name = "sum" if op == "sum" else "mean"
                lib.call(f"keydnn_cuda_{name}_axis2d_forward_{s}", x.data, out, rows, cols, 1)
                return out, rows
            if axis == 0:
                if w == 1 and op == "mean":
                    lib.call(f"keydnn_cuda_mean_axis2d_forward_{s}", x.data, out, rows, cols, 0)
                    return out, cols
                lib.call(f"keydnn_cuda_sum_axis2d_forward_{s}", x.data, out, rows, cols, 0)
                g.allreduce_sum(out, cols, s)
                if op == "mean":
                    lib.call(f"keydnn_cuda_mul_scalar_inplace_{s}", out, self._c(1.0 / (rows * w)), cols)
                return out, cols
            if w == 1 and op == "mean":
                lib.call(f"keydnn_cuda_mean_all_{s}", x.data, out, rows * cols)
                return out, 1
            lib.call(f"keydnn_cuda_sum_all_{s}", x.data, out, rows * cols)
            g.allreduce_sum(out, 1, s)
            if op == "mean":
                lib.call(f"keydnn_cuda_mul_scalar_inplace_{s}", out, self._c(1.0 / (rows * cols * w)), 1)
            return out, 1
        if op != "max":
            raise ValueError(op)
        if axis == 1:
            lib.call(f"keydnn_cuda_max_axis2d_forward_{s}", x.data, out, self.idx.dev_ptr, rows, cols, 1)
            return out, rows
        if axis == 0:
            lib.call(f"keydnn_cuda_max_axis2d_forward_{s}", x.data, out, self.idx.dev_ptr, rows, cols, 0)
            n, span = cols, rows
        else:
            lib.call(f"keydnn_cuda_max_all_forward_{s}", x.data, out, self.idx.dev_ptr, rows * cols)
            n, span = 1, rows * cols
        if w == 1:
            return out, n
        g.allgather(out, self.gather_val.dev_ptr, n * self.dt.itemsize)
        g.allgather(self.idx.dev_ptr, self.gather_idx.dev_ptr, n * 8)
        lib.call(f"keydnn_cuda_argmax_select_{s}", self.gather_val.dev_ptr, self.gather_idx.dev_ptr, w, g.rank, span, n,
                 self.sel_val.data, self.idx_global.dev_ptr, self.idx_local.dev_ptr)
        return self.sel_val.data, n

    # ----------------------------------------------------------------- backward
    def backward(self, op: str, axis: Optional[int], go_ptr: Optional[int] = None) -> int:
        """Gradient of this rank's rows for the last ``forward(op, axis)``; upstream gradient
        defaults to ones.  Returns the device pointer of the (rows, cols) gradient."""
        lib, s = self.lib, self.suf
        rows, cols, w = self.rows, self.cols, self.g.world
        go = self.ones.data if go_ptr is None else go_ptr
        gx = self.gx.data
        if op == "sum":
            if axis is None:
                lib.call(f"keydnn_cuda_sum_backward_fill_{s}", go, gx, rows * cols)
            else:
                lib.call(f"keydnn_cuda_sum_axis2d_backward_{s}", go, gx, rows, cols, axis)
        elif op == "mean":
            if axis is None:
                if w == 1:
                    lib.call(f"keydnn_cuda_mean_backward_fill_{s}", go, gx, rows * cols)
                else:
                    lib.call(f"keydnn_cuda_mul_scalar_{s}", go, self._c(1.0 / (rows * cols * w)), self.go.data, 1)
                    lib.call(f"keydnn_cuda_sum_backward_fill_{s}", self.go.data, gx, rows * cols)
            elif axis == 1 or w == 1:
                lib.call(f"keydnn_cuda_mean_axis2d_backward_{s}", go, gx, rows, cols, axis)
            else:
                lib.call(f"keydnn_cuda_mul_scalar_{s}", go, self._c(1.0 / (rows * w)), self.go.data, cols)
                lib.call(f"keydnn_cuda_sum_axis2d_backward_{s}", self.go.data, gx, rows, cols, 0)
        else:
            local = self.idx.dev_ptr if (w == 1 or axis == 1) else self.idx_local.dev_ptr
            if axis is None:
                lib.call(f"keydnn_cuda_max_all_backward_{s}", go, local, gx, rows * cols)
            else:
                lib.call(f"keydnn_cuda_max_axis2d_backward_ex_{s}", go, local, gx, rows, cols, axis)
        return gx
