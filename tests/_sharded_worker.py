"""One rank of the row-sharded reduction check (spawned by test_multi_gpu.py).

usage: python _sharded_worker.py RANK WORLD ID_FILE OUT_DIR
Each rank owns rows [rank*R, (rank+1)*R) of a seeded global matrix, runs every reduction forward +
backward through ShardedReductions (NCCL inside the library, id exchanged through a file), and writes
its results; the parent compares them with NumPy on the whole matrix."""
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main() -> None:
    rank, world, id_file, out_dir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], Path(sys.argv[4])
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import distributed
    from keydnn_v2_b200.sharded import ExchangeBucket, ShardedReductions

    group = distributed.init_from_file(id_file, rank, world, device=rank, timeout_s=120)
    res = {}
    cases = (("f32", np.float32, 96, 520), ("f64", np.float64, 40, 264))
    # both matrices in ONE shared bucket: a single all-gather moves the partials of both, the sums are formed locally
    shared = ExchangeBucket.for_matrices(group, [(C, dt) for _, dt, _, C in cases])
    joint = {}
    for tag, dt, R, C in cases:
        full = np.random.default_rng(5).standard_normal((R * world, C))
        full = (np.round(full * 4) / 4).astype(dt)          # ties across ranks: the lower rank must win
        full[3, 7] = full[R * world - 2, 7] = 9.0            # same maximum on the first and the last rank
        shard = np.ascontiguousarray(full[rank * R:(rank + 1) * R])
        red = ShardedReductions(kd.Tensor.from_numpy(shard), group)

        def read(ptr, n, shape=None):
            out = np.empty(n if shape is None else shape, dt)
            red.lib.call("keydnn_cuda_memcpy_d2h", out.ctypes.data, ptr, out.nbytes)
            return out

        keys = [(op, ax) for op in ("sum", "mean", "max") for ax in (0, 1, None)]
        # one exchange per reduction, right behind its kernel
        for op, ax in keys:
            ptr, n = red.forward(op, ax)
            red.wait(op, ax)
            res[f"{tag}/{op}/{ax}/y"] = read(ptr, n)
            res[f"{tag}/{op}/{ax}/gx"] = read(red.backward(op, ax), 0, (R, C))
        # all exchanges postponed to one bucket (one all-reduce, one all-gather), then every backward
        outs = {k: red.forward(*k, defer=True) for k in keys}
        red.flush()
        for op, ax in keys:
            res[f"{tag}/bucket/{op}/{ax}/gx"] = read(red.backward(op, ax), 0, (R, C))
        red.finish()
        for (op, ax), (ptr, n) in outs.items():
            res[f"{tag}/bucket/{op}/{ax}/y"] = read(ptr, n)
        # a partial bucket next to finished neighbours: they must keep their values
        part = {k: red.forward(*k, defer=True) for k in (("mean", 0), ("max", None))}
        red.finish()
        for (op, ax), (ptr, n) in part.items():
            res[f"{tag}/partial/{op}/{ax}/y"] = read(ptr, n)
        ptr, n = outs[("sum", 0)]
        res[f"{tag}/partial/sum/0/y"] = read(ptr, n)
        joint[tag] = (ShardedReductions(kd.Tensor.from_numpy(shard), group, bucket=shared), dt, R, C)
    for _ in range(2):                                   # twice: the second round reuses the send buffer
        outs = {(tag, k): red.forward(*k, defer=True) for tag, (red, *_r) in joint.items()
                for k in [(op, ax) for op in ("sum", "mean", "max") for ax in (0, 1, None)]}
        shared.flush()                                   # one collective for both matrices
        for tag, (red, dt, R, C) in joint.items():
            for op in ("sum", "mean", "max"):
                for ax in (0, 1, None):
                    gx = np.empty((R, C), dt)
                    red.lib.call("keydnn_cuda_memcpy_d2h", gx.ctypes.data, red.backward(op, ax), gx.nbytes)
                    res[f"{tag}/shared/{op}/{ax}/gx"] = gx
            red.finish()
        for (tag, (op, ax)), (ptr, n) in outs.items():
            red, dt = joint[tag][0], joint[tag][1]
            y = np.empty(n, dt)
            red.lib.call("keydnn_cuda_memcpy_d2h", y.ctypes.data, ptr, y.nbytes)
            res[f"{tag}/shared/{op}/{ax}/y"] = y
            assert red.result(op, ax) == (ptr, n)
    np.savez(out_dir / f"rank{rank}.npz", **res)
    group.destroy()


if __name__ == "__main__":
    main()
