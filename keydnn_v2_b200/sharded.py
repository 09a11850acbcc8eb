"""Row-sharded reductions: each rank owns ``rows`` consecutive rows of a
(``rows * world``, ``cols``) matrix.

  axis=1           per-row results: local, no exchange.
  axis=0 / None    sum, mean: local partial -> in-place NCCL all-reduce of the (cols,) vector or
                   scalar -> the 1/count scale of the mean is applied after it.
                   max: local (value, first row) pairs -> all-gather -> per-column selection
                   "greater value, else lower rank" (NCCL has no MAXLOC).
  backward         every rank writes its own rows of the gradient; for max only the rank that
                   owns the maximum writes the routed value.

The collectives are tiny (a scalar or one row) and latency-bound, so they run on a second stream:
an event orders each one after the kernel that produced its operand, and the compute stream goes
straight on to the next kernel.  Only a consumer of the reduced value (the max backward, a copy to
the host, ``finish()``) waits for it.  Every (op, axis) has its own result buffers, so nothing on the
compute stream overwrites an operand that is still in flight.  With world == 1 the same calls run
without any collective or second stream.  Buffers are allocated once; a call enqueues work and returns.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import numpy as np

from ._cuda_storage import CudaStorage
from .distributed import Group, single
from .tensor import Tensor, _suffix

Key = Tuple[str, Optional[int]]


class _View:
    """A device address inside a larger allocation (quacks like Tensor.data / CudaStorage.dev_ptr)."""

    def __init__(self, ptr: int) -> None:
        self.data = self.dev_ptr = int(ptr)


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
        isz = self.dt.itemsize
        n_max = max(self.rows, self.cols)
        self._out: Dict[Key, object] = {}
        self._idx: Dict[Key, "_View"] = {}
        self._blk: Dict[Key, Tuple[CudaStorage, int, int]] = {}
        for op in ("sum", "mean", "max"):
            for ax in (0, 1, None):
                n = self.cols if ax == 0 else self.rows if ax == 1 else 1
                if op == "max":
                    # value block and position block side by side: one all-gather moves both
                    voff = (n * isz + 7) // 8 * 8
                    blk = CudaStorage.allocate(voff + n * 8, np.uint8)
                    self._blk[(op, ax)] = (blk, voff, voff + n * 8)
                    self._out[(op, ax)] = _View(blk.dev_ptr)
                    self._idx[(op, ax)] = _View(blk.dev_ptr + voff)
                else:
                    self._out[(op, ax)] = Tensor.empty((n,), self.dt)
        # cross-rank max: gathered candidates and the selection, per axis
        self._gathered = {ax: CudaStorage.allocate(w * self._blk[("max", ax)][2], np.uint8) for ax in (0, None)}
        self._sel = {ax: Tensor.empty((n,), self.dt) for ax, n in ((0, self.cols), (None, 1))}
        self._iglobal = {ax: CudaStorage.allocate(n * 8, np.int64) for ax, n in ((0, self.cols), (None, 1))}
        self._ilocal = {ax: CudaStorage.allocate(n * 8, np.int64) for ax, n in ((0, self.cols), (None, 1))}
        self.ones = Tensor.ones((n_max,), self.dt)             # upstream gradient
        self.go = Tensor.empty((n_max,), self.dt)
        self.gx = Tensor.empty(x.shape, self.dt)
        # second stream + events for the collectives
        self._main = ctypes.c_uint64(0)
        self.lib.call("keydnn_cuda_get_stream", ctypes.byref(self._main))
        self._comm = ctypes.c_uint64(0)
        self._ready = ctypes.c_uint64(0)
        self._done: Dict[Key, int] = {}
        self._pending: set = set()
        if w > 1:
            self.lib.call("keydnn_cuda_stream_create", ctypes.byref(self._comm))
            self.lib.call("keydnn_cuda_event_create", ctypes.byref(self._ready))
            for key in self._out:
                e = ctypes.c_uint64(0)
                self.lib.call("keydnn_cuda_event_create", ctypes.byref(e))
                self._done[key] = e.value

    def _c(self, v: float):
        return ctypes.c_float(v) if self.dt == np.float32 else ctypes.c_double(v)

    # -------------------------------------------------------------- stream hops
    def _on_comm_stream(self, key: Key, fn) -> None:
        """Run `fn` (collective + its small follow-up kernels) on the second stream, after
        everything enqueued so far on the compute stream."""
        lib = self.lib
        lib.call("keydnn_cuda_event_record", self._ready.value)
        lib.call("keydnn_cuda_set_stream", self._comm.value)
        try:
            lib.call("keydnn_cuda_stream_wait_event", self._ready.value)
            fn()
            lib.call("keydnn_cuda_event_record", self._done[key])
        finally:
            lib.call("keydnn_cuda_set_stream", self._main.value)
        self._pending.add(key)

    def wait(self, op: str, axis: Optional[int]) -> None:
        """Later work on the compute stream sees the reduced value of (op, axis)."""
        key = (op, axis)
        if key in self._pending:
            self.lib.call("keydnn_cuda_stream_wait_event", self._done[key])
            self._pending.discard(key)

    def finish(self) -> None:
        """Order everything outstanding on the second stream before later compute-stream work."""
        for key in list(self._pending):
            self.wait(*key)

    # ------------------------------------------------------------------ forward
    def forward(self, op: str, axis: Optional[int]) -> Tuple[int, int]:
        """Runs one reduction; returns (device pointer, element count) of the result.  At
        world > 1 the value of an axis-0 / all-axes result is complete after ``wait(op, axis)``."""
        lib, x, s, g = self.lib, self.x, self.suf, self.g
        rows, cols, w = self.rows, self.cols, self.g.world
        key = (op, axis)
        self.wait(op, axis)                      # the buffers of this key are about to be rewritten
        out = self._out[key].data
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
                n, count = cols, rows * w
            else:
                if w == 1 and op == "mean":
                    lib.call(f"keydnn_cuda_mean_all_{s}", x.data, out, rows * cols)
                    return out, 1
                lib.call(f"keydnn_cuda_sum_all_{s}", x.data, out, rows * cols)
                n, count = 1, rows * cols * w
            if w > 1:
                def exchange() -> None:
                    g.allreduce_sum(out, n, s)
                    if op == "mean":
                        lib.call(f"keydnn_cuda_mul_scalar_inplace_{s}", out, self._c(1.0 / count), n)

                self._on_comm_stream(key, exchange)
            return out, n
        if op != "max":
            raise ValueError(op)
        idx = self._idx[key].dev_ptr
        if axis == 1:
            lib.call(f"keydnn_cuda_max_axis2d_forward_{s}", x.data, out, idx, rows, cols, 1)
            return out, rows
        if axis == 0:
            lib.call(f"keydnn_cuda_max_axis2d_forward_{s}", x.data, out, idx, rows, cols, 0)
            n, span = cols, rows
        else:
            lib.call(f"keydnn_cuda_max_all_forward_{s}", x.data, out, idx, rows * cols)
            n, span = 1, rows * cols
        if w == 1:
            return out, n

        _, voff, blk_bytes = self._blk[key]
        gathered = self._gathered[axis].dev_ptr

        def exchange_max() -> None:
            g.allgather(out, gathered, blk_bytes)
            lib.call(f"keydnn_cuda_argmax_select_{s}", gathered, gathered + voff, w, g.rank, span, n,
                     blk_bytes // self.dt.itemsize, blk_bytes // 8, self._sel[axis].data,
                     self._iglobal[axis].dev_ptr, self._ilocal[axis].dev_ptr)

        self._on_comm_stream(key, exchange_max)
        return self._sel[axis].data, n

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
            if w == 1 or axis == 1:
                local = self._idx[(op, axis)].dev_ptr
            else:
                self.wait(op, axis)              # the owner of each maximum is known after the exchange
                local = self._ilocal[axis].dev_ptr
            if axis is None:
                lib.call(f"keydnn_cuda_max_all_backward_{s}", go, local, gx, rows * cols)
            else:
                lib.call(f"keydnn_cuda_max_axis2d_backward_ex_{s}", go, local, gx, rows, cols, axis)
        return gx
