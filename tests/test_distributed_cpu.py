"""Host-side logic of the multi-GPU layer with world_size 2 on CPU: the NCCL id must travel from
rank 0 to every rank (through torch.distributed/gloo and through a file) and each rank must call
keydnn_nccl_init with its own rank.  The native library is replaced by a recorder: no GPU, no NCCL."""
from __future__ import annotations

import multiprocessing as mp
import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]


class FakeNative:
    def __init__(self, rank):
        self.rank, self.calls = rank, []

    def call(self, name, *args):
        if name == "keydnn_nccl_unique_id":
            args[0].raw = bytes([7 + self.rank]) * 128           # rank 0's id is 0x07 * 128
        self.calls.append((name, tuple(a.raw if hasattr(a, "raw") else a for a in args)))


def _gloo_rank(rank, world, port, q):
    sys.path.insert(0, str(REPO))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    from keydnn_v2_b200 import distributed

    dist.init_process_group("gloo", rank=rank, world_size=world)
    fake = FakeNative(rank)

    def exchange(b):
        box = [b]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    g = distributed.init(rank, world, exchange, device=None, native=fake)
    q.put((rank, g.rank, g.world, fake.calls))
    dist.destroy_process_group()


def _file_rank(rank, world, path, q):
    sys.path.insert(0, str(REPO))
    from keydnn_v2_b200 import distributed

    fake = FakeNative(rank)
    import keydnn_v2_b200.distributed as d

    d.load = lambda: fake
    g = distributed.init_from_file(path, rank, world, timeout_s=30)
    q.put((rank, g.rank, g.world, fake.calls))


def _check(results, world):
    assert sorted(r[0] for r in results) == list(range(world))
    for rank, grank, gworld, calls in results:
        assert (grank, gworld) == (rank, world)
        init = [c for c in calls if c[0] == "keydnn_nccl_init"]
        assert len(init) == 1
        ident, w, r = init[0][1]
        assert ident == bytes([7]) * 128 and (w, r) == (world, rank)       # everybody got rank 0's id
        assert ("keydnn_nccl_unique_id" in [c[0] for c in calls]) == (rank == 0)


def test_id_exchange_over_gloo_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    ps = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    results = [q.get(timeout=120) for _ in ps]
    [p.join(timeout=60) for p in ps]
    _check(results, 2)


def test_id_exchange_over_a_file_world_size_2(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_file_rank, args=(r, 2, str(tmp_path / "id"), q)) for r in (1, 0)]   # rank 1 first: it waits
    [p.start() for p in ps]
    results = [q.get(timeout=60) for _ in ps]
    [p.join(timeout=30) for p in ps]
    _check(results, 2)


def test_missing_rank0_times_out_instead_of_hanging(tmp_path):
    from keydnn_v2_b200 import distributed

    with pytest.raises(TimeoutError):
        distributed.init_from_file(tmp_path / "never", 1, 2, timeout_s=0.3, device=None)


def test_world_size_1_needs_no_nccl():
    from keydnn_v2_b200 import distributed

    fake = FakeNative(0)
    g = distributed.init(0, 1, lambda b: b, native=fake)
    assert (g.rank, g.world) == (0, 1) and fake.calls == []
    g.allreduce_sum(1234, 8, "f32")
    assert fake.calls == []
