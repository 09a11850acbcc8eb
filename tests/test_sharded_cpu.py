"""The row-sharded reductions with world_size 2 and 8 on CPU (gloo): the host-side logic of `keydnn_v2_b200.sharded` -
buffer layout inside the shared exchange bucket, offsets and strides handed to the selection / rank-order-sum
kernels, which collective moves what, which results are complete when - driven against a stand-in for the native
library that keeps "device" memory in host arrays, computes every called entry with NumPy and moves the
collectives through torch.distributed.  No GPU, no NCCL; the kernels themselves are checked on the GPU
(tests/test_reduce_gpu.py, tests/test_multi_gpu.py)."""
from __future__ import annotations

import ctypes
import multiprocessing as mp
import os
import sys
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[1]


class HostNative:
    """Every `keydnn_*` entry the sharded reductions call, on host memory."""

    def __init__(self, dist):
        self.dist, self.rank, self.world = dist, dist.get_rank(), dist.get_world_size()
        self.blocks, self.calls, self._next = {}, [], 1
        self.path = "host stand-in"

    # -- memory ------------------------------------------------------------------------------------
    def view(self, ptr, n, dtype):
        dt = np.dtype(dtype)
        return np.frombuffer((ctypes.c_char * (n * dt.itemsize)).from_address(int(ptr)), dtype=dt, count=n)

    def raw(self, name):
        return lambda *a: (self.call(name, *a), 0)[1]

    def has(self, name):
        return True

    def call(self, name, *a):
        self.calls.append(name)
        a = [x.value if isinstance(x, (ctypes.c_uint64, ctypes.c_int64, ctypes.c_size_t, ctypes.c_float, ctypes.c_double,
                                       ctypes.c_int)) else x for x in a]
        dt = np.float32 if name.endswith("_f32") else np.float64
        if name == "keydnn_cuda_malloc":
            buf = np.zeros(max(int(a[1]), 8) + 64, np.uint8)
            addr = (buf.ctypes.data + 63) // 64 * 64
            self.blocks[addr] = buf
            a[0]._obj.value = addr
        elif name == "keydnn_cuda_free":
            self.blocks.pop(int(a[0]), None)
        elif name == "keydnn_cuda_memset":
            self.view(a[0], a[2], np.uint8)[:] = a[1]
        elif name in ("keydnn_cuda_memcpy_h2d", "keydnn_cuda_memcpy_d2h", "keydnn_cuda_memcpy_d2d"):
            ctypes.memmove(int(a[0]), int(a[1]), int(a[2]))
        elif name in ("keydnn_cuda_stream_create", "keydnn_cuda_event_create"):
            a[0]._obj.value = 1000 + self._next
            self._next += 1
        elif name == "keydnn_cuda_get_stream":
            a[0]._obj.value = 0
        elif name in ("keydnn_cuda_set_stream", "keydnn_cuda_event_record", "keydnn_cuda_stream_wait_event",
                      "keydnn_cuda_synchronize", "keydnn_cuda_set_device"):
            pass
        elif name.startswith("keydnn_cuda_fill_"):
            self.view(a[0], a[1], dt)[:] = a[2]
        # -- the local kernels ---------------------------------------------------------------------
        elif name.startswith(("keydnn_cuda_sum_axis2d_forward_", "keydnn_cuda_mean_axis2d_forward_")):
            x, y, rows, cols, axis = a
            m = self.view(x, rows * cols, dt).reshape(rows, cols).astype(np.float64)
            r = m.sum(axis) if "sum_axis2d" in name else m.mean(axis)
            self.view(y, r.size, dt)[:] = r
        elif name.startswith(("keydnn_cuda_sum_all_", "keydnn_cuda_mean_all_")):
            v = self.view(a[0], a[2], dt).astype(np.float64)
            self.view(a[1], 1, dt)[0] = v.sum() if "sum_all" in name else v.mean()
        elif name.startswith("keydnn_cuda_max_axis2d_forward_"):
            x, y, idx, rows, cols, axis = a
            m = self.view(x, rows * cols, dt).reshape(rows, cols)
            self.view(y, m.shape[1 - axis], dt)[:] = m.max(axis)
            self.view(idx, m.shape[1 - axis], np.int64)[:] = m.argmax(axis)
        elif name.startswith("keydnn_cuda_max_all_forward_"):
            v = self.view(a[0], a[3], dt)
            self.view(a[1], 1, dt)[0] = v.max()
            self.view(a[2], 1, np.int64)[0] = v.argmax()
        elif name.startswith("keydnn_cuda_mul_scalar_inplace_"):
            self.view(a[0], a[2], dt)[:] *= dt(a[1])
        elif name.startswith("keydnn_cuda_rank_sum_"):
            blocks, world, stride, n, out, sb, se, sc, nseg = a
            acc = np.zeros(n, np.float64)
            for r in range(world):
                acc += self.view(blocks + r * stride * np.dtype(dt).itemsize, n, dt)
            res = acc.astype(dt)
            for k in range(nseg):
                res[sb[k]:se[k]] *= dt(sc[k])
            self.view(out, n, dt)[:] = res
        elif name.startswith("keydnn_cuda_argmax_select_"):
            vals, idx, world, rank, span, n, vs, istr, ov, og, ol = a
            isz = np.dtype(dt).itemsize
            best, g, owner = np.full(n, -np.inf), np.zeros(n, np.int64), np.zeros(n, np.int64)
            for r in range(world):
                v = self.view(vals + r * vs * isz, n, dt)
                i = self.view(idx + r * istr * 8, n, np.int64)
                win = v > best
                best, g, owner = np.where(win, v, best), np.where(win, r * span + i, g), np.where(win, r, owner)
            self.view(ov, n, dt)[:] = best
            self.view(og, n, np.int64)[:] = g
            self.view(ol, n, np.int64)[:] = np.where(owner == rank, g - rank * span, -1)
        # -- collectives through gloo --------------------------------------------------------------
        elif name == "keydnn_nccl_allgather":
            import torch

            send = torch.from_numpy(self.view(a[0], a[2], np.uint8).copy())
            parts = [torch.empty_like(send) for _ in range(self.world)]
            self.dist.all_gather(parts, send)
            self.view(a[1], a[2] * self.world, np.uint8)[:] = torch.cat(parts).numpy()
        elif name.startswith("keydnn_nccl_allreduce_sum_"):
            import torch

            t = torch.from_numpy(self.view(a[0], a[1], dt).copy())
            self.dist.all_reduce(t)
            self.view(a[0], a[1], dt)[:] = t.numpy()
        else:
            raise AssertionError(f"the stand-in has no {name}")


def _rank(rank, world, port, q):
    sys.path.insert(0, str(REPO))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    import keydnn_v2_b200._cuda_storage as storage
    from keydnn_v2_b200.distributed import Group
    from keydnn_v2_b200.sharded import ExchangeBucket, ShardedReductions
    from keydnn_v2_b200.tensor import Tensor

    host = HostNative(dist)
    storage.load = lambda: host                       # every allocation of this process goes to the stand-in
    group = Group(rank, world, host)
    cases = [("f32", np.float32, 24, 40), ("f64", np.float64, 16, 13)]        # 13 columns: unpadded widths
    wholes, out = {}, {}
    try:
        for mode in ("shared bucket", "one matrix at a time"):
            bucket = ExchangeBucket.for_matrices(group, [(c, dt) for _, dt, _, c in cases]) if mode == "shared bucket" else None
            reds = {}
            for tag, dt, R, C in cases:
                whole = np.random.default_rng(3).standard_normal((R * world, C)).astype(dt)
                whole[1, 2] = whole[R * world - 1, 2] = 8.0        # a tie across the ranks: the lower global row wins
                wholes[tag] = whole
                reds[tag] = ShardedReductions(Tensor.from_numpy(np.ascontiguousarray(whole[rank * R:(rank + 1) * R])), group,
                                              bucket=bucket)
            keys = [(op, ax) for op in ("sum", "mean", "max") for ax in (0, 1, None)]
            for _ in range(2):                                   # the second round reuses every buffer
                before = len(host.calls)
                for red in reds.values():
                    for k in keys:
                        red.forward(*k, defer=True)
                for red in reds.values():
                    red.flush()
                for red in reds.values():
                    red.finish()
                moved = [c for c in host.calls[before:] if c.startswith("keydnn_nccl_")]
                out[f"{mode}/collectives"] = moved
            for tag, dt, R, C in cases:
                red = reds[tag]
                for op, ax in keys:
                    ptr, n = red.result(op, ax)
                    out[f"{mode}/{tag}/{op}/{ax}"] = host.view(ptr, n, dt).copy()
                out[f"{mode}/{tag}/argmax0"] = host.view(red._iglobal[0].dev_ptr, C, np.int64).copy()
                out[f"{mode}/{tag}/argmax_all"] = host.view(red._iglobal[None].dev_ptr, 1, np.int64).copy()
                out[f"{mode}/{tag}/local0"] = host.view(red._ilocal[0].dev_ptr, C, np.int64).copy()
        q.put((rank, out, {k: v for k, v in wholes.items()}))
    finally:
        dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("world", [2, 8])
def test_sharded_reductions_over_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() + 7 * world) % 1500
    ps = [ctx.Process(target=_rank, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    got = sorted((q.get(timeout=400) for _ in ps), key=lambda t: t[0])
    [p.join(timeout=60) for p in ps]
    for rank, out, wholes in got:
        # one byte all-gather per flush for BOTH matrices with the shared bucket; an all-reduce and an all-gather per matrix without
        assert out["shared bucket/collectives"] == ["keydnn_nccl_allgather"]
        assert sorted(out["one matrix at a time/collectives"]) == ["keydnn_nccl_allgather"] * 2 + [
            "keydnn_nccl_allreduce_sum_f32", "keydnn_nccl_allreduce_sum_f64"]
        for mode in ("shared bucket", "one matrix at a time"):
            for tag, whole in wholes.items():
                R = whole.shape[0] // world
                tol = dict(rtol=1e-5, atol=1e-5) if whole.dtype == np.float32 else dict(rtol=1e-12, atol=1e-12)
                w64 = whole.astype(np.float64)
                mine = slice(rank * R, (rank + 1) * R)
                np.testing.assert_allclose(out[f"{mode}/{tag}/sum/0"], w64.sum(0), **tol)
                np.testing.assert_allclose(out[f"{mode}/{tag}/mean/0"], w64.mean(0), **tol)
                np.testing.assert_allclose(out[f"{mode}/{tag}/sum/None"], [w64.sum()], **tol)
                np.testing.assert_allclose(out[f"{mode}/{tag}/mean/None"], [w64.mean()], **tol)
                np.testing.assert_allclose(out[f"{mode}/{tag}/sum/1"], w64[mine].sum(1), **tol)
                np.testing.assert_allclose(out[f"{mode}/{tag}/mean/1"], w64[mine].mean(1), **tol)
                np.testing.assert_array_equal(out[f"{mode}/{tag}/max/0"], whole.max(0))
                np.testing.assert_array_equal(out[f"{mode}/{tag}/max/None"], [whole.max()])
                np.testing.assert_array_equal(out[f"{mode}/{tag}/max/1"], whole[mine].max(1))
                np.testing.assert_array_equal(out[f"{mode}/{tag}/argmax0"], whole.argmax(0))
                np.testing.assert_array_equal(out[f"{mode}/{tag}/argmax_all"], [whole.argmax()])
                owner = whole.argmax(0) // R
                np.testing.assert_array_equal(out[f"{mode}/{tag}/local0"], np.where(owner == rank, whole.argmax(0) - rank * R, -1))
