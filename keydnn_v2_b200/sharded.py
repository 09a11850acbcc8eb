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

``forward(..., defer=True)`` postpones the exchange to ``flush()``, which moves everything postponed with
ONE all-reduce (the sum / mean partials of axis 0 and of all axes lie side by side in one buffer) and ONE
all-gather (both max candidate blocks lie side by side): two latency-bound collectives per step and matrix
instead of six, issued where the caller chooses - e.g. after the last forward kernel, so that they run
under the streaming backward kernels and not next to the one-wave reduction kernels whose grids fill
every SM exactly.

``ExchangeBucket`` goes one step further: several ``ShardedReductions`` (say an fp32 and an fp64 matrix) place
their partial blocks in ONE send buffer, and a flush is ONE byte all-gather for all of them followed by local
kernels: the sums are formed from the gathered blocks in rank order (``keydnn_cuda_rank_sum``: double
accumulation, one rounding, the mean's 1/count folded in), the maxima by the same selection as before.  One
latency-bound collective per step instead of four, and the sum no longer depends on the order a collective
library happens to add in.
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


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class ExchangeBucket:
    """One send buffer shared by several ``ShardedReductions`` and one all-gather per ``flush()``.

    ``nbytes`` must cover the members' needs (``ExchangeBucket.bytes_for(cols, dtype)`` each).  Create the bucket,
    pass it to every ``ShardedReductions(x, group, bucket=bucket)``, run the forward reductions with
    ``defer=True`` and call ``flush()`` on the bucket (or on any member) once: everything postponed by all
    members crosses the ranks together."""

    def __init__(self, group: Group, nbytes: int) -> None:
        self.g, self.lib = group, group.native
        self.total = _align(int(nbytes))
        self.used = 0
        self.members: list = []
        self.send = CudaStorage.allocate(self.total, np.uint8)
        self.recv = CudaStorage.allocate(self.total * group.world, np.uint8)
        self.lib.call("keydnn_cuda_memset", self.send.dev_ptr, 0, self.total)
        self._main = ctypes.c_uint64(0)
        self.lib.call("keydnn_cuda_get_stream", ctypes.byref(self._main))
        self._comm, self._ready, self._done = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_uint64(0)
        if group.world > 1:
            self.lib.call("keydnn_cuda_stream_create", ctypes.byref(self._comm))
            self.lib.call("keydnn_cuda_event_create", ctypes.byref(self._ready))
            self.lib.call("keydnn_cuda_event_create", ctypes.byref(self._done))

    @staticmethod
    def bytes_for(cols: int, dtype) -> int:
        """Bytes one (rows, cols) matrix of `dtype` needs in the bucket: its sum block and its max block."""
        isz = np.dtype(dtype).itemsize
        cpad = (cols + 3) // 4 * 4
        max_bytes = 0
        for n in (cols, 1):
            max_bytes += (n * isz + 7) // 8 * 8 + n * 8
        return _align((2 * cpad + 2) * isz) + _align(max_bytes)

    @classmethod
    def for_matrices(cls, group: Group, shapes) -> "ExchangeBucket":
        """`shapes`: (cols, dtype) of every matrix that will join."""
        return cls(group, sum(cls.bytes_for(c, d) for c, d in shapes))

    def take(self, nbytes: int) -> int:
        """Offset of a fresh 256-byte aligned piece of the send buffer."""
        off = self.used
        if off + _align(nbytes) > self.total:
            raise ValueError("ExchangeBucket is too small for its members")
        self.used += _align(nbytes)
        return off

    def flush(self) -> None:
        todo = [(m, m._take_deferred()) for m in self.members]
        todo = [(m, items) for m, items in todo if items]
        if not todo:
            return
        lib = self.lib
        lib.call("keydnn_cuda_event_record", self._ready.value)
        lib.call("keydnn_cuda_set_stream", self._comm.value)
        try:
            lib.call("keydnn_cuda_stream_wait_event", self._ready.value)
            self.g.allgather(self.send.dev_ptr, self.recv.dev_ptr, self.total)
            for m, items in todo:
                m._after_gather(items, self.recv.dev_ptr, self.total)
            lib.call("keydnn_cuda_event_record", self._done.value)
        finally:
            lib.call("keydnn_cuda_set_stream", self._main.value)
        for m, items in todo:
            for key, _ in items:
                m._pending.add(key)
                m._wait_for[key] = self._done.value


class ShardedReductions:
    def __init__(self, x: Tensor, group: Optional[Group] = None, bucket: Optional[ExchangeBucket] = None) -> None:
        if x.ndim != 2:
            raise ValueError("ShardedReductions needs a 2-D local shard")
        self.x = x
        self.g = group or single(x.native)
        self.lib = x.native
        self.bucket = bucket if (bucket is not None and self.g.world > 1) else None
        self.rows, self.cols = x.shape
        self.dt = x.dtype
        self.suf = _suffix(self.dt)
        w = self.g.world
        isz = self.dt.itemsize
        n_max = max(self.rows, self.cols)
        self._out: Dict[Key, object] = {}
        self._idx: Dict[Key, "_View"] = {}
        self._blk: Dict[Key, Tuple[object, int, int]] = {}
        # the four partials that cross ranks share one buffer: [sum ax0 | mean ax0 | sum all | mean all]
        cpad = (self.cols + 3) // 4 * 4
        self._cpad = cpad
        self._sum_count = 2 * cpad + 2
        if self.bucket is not None:
            # partials go straight into the shared send buffer; the reduced values land in a buffer of their own
            self._sum_off = self.bucket.take(self._sum_count * isz)
            self._sumblk = _View(self.bucket.send.dev_ptr + self._sum_off)
            self._sumres = Tensor.empty((self._sum_count,), self.dt)
            self.lib.call("keydnn_cuda_memset", self._sumres.data, 0, self._sum_count * isz)
            self.bucket.members.append(self)
        else:
            self._sumblk = Tensor.empty((self._sum_count,), self.dt)
            self._sumres = self._sumblk
            self.lib.call("keydnn_cuda_memset", self._sumblk.data, 0, self._sum_count * isz)
        self._sum_pos = {("sum", 0): 0, ("mean", 0): cpad, ("sum", None): 2 * cpad, ("mean", None): 2 * cpad + 1}
        self._res: Dict[Key, "_View"] = {}
        for key, pos in self._sum_pos.items():
            self._out[key] = _View(self._sumblk.data + pos * isz)
            self._res[key] = _View(self._sumres.data + pos * isz)
        for op in ("sum", "mean"):
            self._out[(op, 1)] = Tensor.empty((self.rows,), self.dt)
        # max: value block and position block side by side, and the two blocks that cross ranks (axis 0, all
        # axes) side by side as well: one all-gather moves everything
        sizes = {}
        for ax in (0, None, 1):
            n = self.cols if ax == 0 else self.rows if ax == 1 else 1
            voff = (n * isz + 7) // 8 * 8
            sizes[ax] = (voff, voff + n * 8)
        self._maxblk_bytes = sizes[0][1] + sizes[None][1]
        if self.bucket is not None:
            self._max_off = self.bucket.take(self._maxblk_bytes)
            self._maxblk = _View(self.bucket.send.dev_ptr + self._max_off)
        else:
            self._maxblk = CudaStorage.allocate(self._maxblk_bytes, np.uint8)
            self.lib.call("keydnn_cuda_memset", self._maxblk.dev_ptr, 0, self._maxblk_bytes)
        own1 = CudaStorage.allocate(sizes[1][1], np.uint8)
        for ax, base, owner in ((0, self._maxblk.dev_ptr, self._maxblk), (None, self._maxblk.dev_ptr + sizes[0][1], self._maxblk),
                                (1, own1.dev_ptr, own1)):
            voff, nbytes = sizes[ax]
            self._blk[("max", ax)] = (owner, voff, nbytes)
            self._out[("max", ax)] = _View(base)
            self._idx[("max", ax)] = _View(base + voff)
        # cross-rank max: gathered candidates (per axis, and of both blocks at once) and the selection
        self._gathered = {ax: CudaStorage.allocate(w * self._blk[("max", ax)][2], np.uint8) for ax in (0, None)}
        self._gathered_all = CudaStorage.allocate(w * self._maxblk_bytes, np.uint8) if self.bucket is None else None
        self._deferred: list = []
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
            for key in list(self._out) + [("bucket", None)]:
                e = ctypes.c_uint64(0)
                self.lib.call("keydnn_cuda_event_create", ctypes.byref(e))
                self._done[key] = e.value
        self._wait_for: Dict[Key, int] = {}      # pending key -> the event that completes it

    def _c(self, v: float):
        return ctypes.c_float(v) if self.dt == np.float32 else ctypes.c_double(v)

    # -------------------------------------------------------------- stream hops
    def _on_comm_stream(self, keys, fn, event_key: Optional[Key] = None) -> None:
        """Run `fn` (collective + its small follow-up kernels) on the second stream, after
        everything enqueued so far on the compute stream; `keys` complete with it."""
        lib = self.lib
        event = self._done[event_key if event_key is not None else keys[0]]
        lib.call("keydnn_cuda_event_record", self._ready.value)
        lib.call("keydnn_cuda_set_stream", self._comm.value)
        try:
            lib.call("keydnn_cuda_stream_wait_event", self._ready.value)
            fn()
            lib.call("keydnn_cuda_event_record", event)
        finally:
            lib.call("keydnn_cuda_set_stream", self._main.value)
        for key in keys:
            self._pending.add(key)
            self._wait_for[key] = event

    def wait(self, op: str, axis: Optional[int]) -> None:
        """Later work on the compute stream sees the reduced value of (op, axis)."""
        key = (op, axis)
        if any(k == key for k, _ in self._deferred):
            self.flush()
        if key in self._pending:
            event = self._wait_for.pop(key)
            self.lib.call("keydnn_cuda_stream_wait_event", event)
            self._pending.discard(key)
            for other in [k for k, e in self._wait_for.items() if e == event]:      # same collective: done as well
                self._pending.discard(other)
                del self._wait_for[other]

    def finish(self) -> None:
        """Order everything outstanding on the second stream before later compute-stream work."""
        self.flush()
        for key in list(self._pending):
            self.wait(*key)

    def flush(self) -> None:
        """Exchange everything ``forward(..., defer=True)`` postponed: one all-reduce over the shared sum buffer,
        one all-gather over the shared max block, the mean scales and the selections behind them."""
        if self.bucket is not None:
            self.bucket.flush()
            return
        if not self._deferred:
            return
        todo, self._deferred = self._deferred, []
        lib, s, g, w = self.lib, self.suf, self.g, self.g.world
        isz = self.dt.itemsize

        def exchange() -> None:
            sums = [(k, meta) for k, meta in todo if k[0] != "max"]
            maxes = [(k, meta) for k, meta in todo if k[0] == "max"]
            if len(sums) == 4:
                g.allreduce_sum(self._sumblk.data, self._sum_count, s)      # all four partials at once
            else:
                for (op, ax), (n, _) in sums:                               # never re-reduce a finished neighbour
                    g.allreduce_sum(self._out[(op, ax)].data, n, s)
            if sums:
                for (op, ax), (n, count) in sums:
                    if op == "mean":
                        lib.call(f"keydnn_cuda_mul_scalar_inplace_{s}", self._out[(op, ax)].data, self._c(1.0 / count), n)
            if maxes:
                total = self._maxblk_bytes
                gathered = self._gathered_all.dev_ptr
                g.allgather(self._maxblk.dev_ptr, gathered, total)
                for (op, ax), (n, span) in maxes:
                    base = gathered + (self._out[(op, ax)].data - self._maxblk.dev_ptr)
                    voff = self._blk[(op, ax)][1]
                    lib.call(f"keydnn_cuda_argmax_select_{s}", base, base + voff, w, g.rank, span, n, total // isz, total // 8,
                             self._sel[ax].data, self._iglobal[ax].dev_ptr, self._ilocal[ax].dev_ptr)

        self._on_comm_stream([k for k, _ in todo], exchange, ("bucket", None))

    # ------------------------------------------------------- shared-bucket exchange
    def _take_deferred(self) -> list:
        todo, self._deferred = self._deferred, []
        return todo

    def _after_gather(self, items, recv: int, total: int) -> None:
        """Local kernels behind the bucket's all-gather (`recv` holds world blocks of `total` bytes): sums of the
        gathered partials in rank order with the mean scales folded in, selections of the gathered maxima."""
        lib, s, w, isz = self.lib, self.suf, self.g.world, self.dt.itemsize
        i64, ct = ctypes.c_int64, (ctypes.c_float if self.dt == np.float32 else ctypes.c_double)
        sums = [(k, meta) for k, meta in items if k[0] != "max"]
        maxes = [(k, meta) for k, meta in items if k[0] == "max"]
        base = recv + self._sum_off
        if len(sums) == 4:
            scales = {k: 1.0 / count for k, (n, count) in sums if k[0] == "mean"}
            segs = [(self._sum_pos[k], self._sum_pos[k] + n, scales[k]) for k, (n, _) in sums if k[0] == "mean"]
            lib.call(f"keydnn_cuda_rank_sum_{s}", base, w, total // isz, self._sum_count, self._sumres.data,
                     (i64 * len(segs))(*[a for a, _, _ in segs]), (i64 * len(segs))(*[b for _, b, _ in segs]),
                     (ct * len(segs))(*[c for _, _, c in segs]), len(segs))
        else:
            for k, (n, count) in sums:                                 # never touch a finished neighbour
                off = self._sum_pos[k] * isz
                seg = ((i64 * 1)(0), (i64 * 1)(n), (ct * 1)(1.0 / count), 1) if k[0] == "mean" else (None, None, None, 0)
                lib.call(f"keydnn_cuda_rank_sum_{s}", base + off, w, total // isz, n, self._sumres.data + off, *seg)
        for (op, ax), (n, span) in maxes:
            vbase = recv + self._max_off + (self._out[(op, ax)].data - self._maxblk.dev_ptr)
            voff = self._blk[(op, ax)][1]
            lib.call(f"keydnn_cuda_argmax_select_{s}", vbase, vbase + voff, w, self.g.rank, span, n, total // isz, total // 8,
                     self._sel[ax].data, self._iglobal[ax].dev_ptr, self._ilocal[ax].dev_ptr)

    def result(self, op: str, axis: Optional[int]) -> Tuple[int, int]:
        """(device pointer, element count) of the complete value of (op, axis) (after ``wait`` / ``finish``)."""
        n = self.rows if axis == 1 else self.cols if axis == 0 else 1
        if op == "max":
            return (self._sel[axis].data if (self.g.world > 1 and axis != 1) else self._out[(op, axis)].data), n
        if axis == 1:
            return self._out[(op, axis)].data, n
        return (self._res[(op, axis)].data if self.bucket is not None else self._out[(op, axis)].data), n

    # ------------------------------------------------------------------ forward
    def forward(self, op: str, axis: Optional[int], defer: bool = False) -> Tuple[int, int]:
        """Runs one reduction; returns (device pointer, element count) of the result.  At
        world > 1 the value of an axis-0 / all-axes result is complete after ``wait(op, axis)``;
        with ``defer`` its exchange is postponed to the next ``flush()`` (or the first ``wait`` for it)."""
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
            if self.bucket is not None:
                self._deferred.append((key, (n, count)))
                if not defer:
                    self.bucket.flush()
                return self._res[key].data, n
            if w > 1 and defer:
                self._deferred.append((key, (n, count)))
            elif w > 1:
                def exchange() -> None:
                    g.allreduce_sum(out, n, s)
                    if op == "mean":
                        lib.call(f"keydnn_cuda_mul_scalar_inplace_{s}", out, self._c(1.0 / count), n)

                self._on_comm_stream([key], exchange)
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

        if defer or self.bucket is not None:
            self._deferred.append((key, (n, span)))
            if not defer:
                self.bucket.flush()
            return self._sel[axis].data, n
        _, voff, blk_bytes = self._blk[key]
        gathered = self._gathered[axis].dev_ptr

        def exchange_max() -> None:
            g.allgather(out, gathered, blk_bytes)
            lib.call(f"keydnn_cuda_argmax_select_{s}", gathered, gathered + voff, w, g.rank, span, n,
                     blk_bytes // self.dt.itemsize, blk_bytes // 8, self._sel[axis].data,
                     self._iglobal[axis].dev_ptr, self._ilocal[axis].dev_ptr)

        self._on_comm_stream([key], exchange_max)
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
