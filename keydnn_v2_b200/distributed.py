"""One process per GPU: NCCL communicator inside ``libkeydnn_b200.so``.

The reference registers its CUDA control paths for ``Device("cuda:0")`` only
(``src/keydnn/domain/device/_device.py:124-155``) and has no collective of any kind, so a
multi-GPU job is N processes, each driving one GPU, with the 128-byte NCCL id handed from rank 0
to the others over whatever the launcher offers (a ``torch.distributed`` group, or a file).
"""
from __future__ import annotations

import ctypes
import os
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Optional

from ._native import Native, load


@dataclass
class Group:
    rank: int
    world: int
    native: Native

    def allreduce_sum(self, ptr: int, count: int, dtype_suffix: str) -> None:
        if self.world > 1:
            self.native.call(f"keydnn_nccl_allreduce_sum_{dtype_suffix}", ptr, count)

    def allgather(self, send_ptr: int, recv_ptr: int, nbytes: int) -> None:
        if self.world == 1:
            self.native.call("keydnn_cuda_memcpy_d2d", recv_ptr, send_ptr, nbytes)
        else:
            self.native.call("keydnn_nccl_allgather", send_ptr, recv_ptr, nbytes)

    def broadcast(self, ptr: int, nbytes: int, root: int = 0) -> None:
        if self.world > 1:
            self.native.call("keydnn_nccl_broadcast", ptr, nbytes, root)

    def destroy(self) -> None:
        self.native.call("keydnn_nccl_destroy")


def single(native: Optional[Native] = None) -> Group:
    return Group(0, 1, native or load())


def init(rank: int, world: int, exchange: Callable[[Optional[bytes]], bytes], *, device: Optional[int] = None,
         native: Optional[Native] = None) -> Group:
    """``exchange(id_or_None)`` must return rank 0's bytes on every rank (rank 0 passes the id)."""
    native = native or load()
    if device is not None:
        native.call("keydnn_cuda_set_device", int(device))
    if world == 1:
        return Group(0, 1, native)
    buf = ctypes.create_string_buffer(128)
    if rank == 0:
        native.call("keydnn_nccl_unique_id", buf)
        ident = exchange(bytes(buf.raw))
    else:
        ident = exchange(None)
    if len(ident) != 128:
        raise RuntimeError("NCCL id exchange returned a wrong size")
    native.call("keydnn_nccl_init", ctypes.create_string_buffer(ident, 128), world, rank)
    return Group(rank, world, native)


def init_from_torch(device: Optional[int] = None) -> Group:
    """Rank / world and the id exchange come from an initialised ``torch.distributed`` group."""
    import torch.distributed as dist

    rank, world = dist.get_rank(), dist.get_world_size()

    def exchange(b: Optional[bytes]) -> bytes:
        box = [b]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    return init(rank, world, exchange, device=device)


def init_from_file(path: str | os.PathLike, rank: int, world: int, *, device: Optional[int] = None,
                   timeout_s: float = 60.0) -> Group:
    """Rank 0 writes the id to `path`; the others wait for it (bounded) and read it."""
    path = Path(path)

    def exchange(b: Optional[bytes]) -> bytes:
        if b is not None:
            tmp = path.with_suffix(".tmp")
            tmp.write_bytes(b)
            tmp.replace(path)
            return b
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            if path.exists() and path.stat().st_size == 128:
                return path.read_bytes()
            time.sleep(0.05)
        raise TimeoutError(f"rank {rank}: no NCCL id at {path} after {timeout_s}s (did rank 0 start?)")

    return init(rank, world, exchange, device=device)
