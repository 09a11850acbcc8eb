"""One rank of the data-parallel training check (spawned by test_multi_gpu.py).

usage: python _dp_worker.py RANK WORLD ID_FILE OUT_DIR
Every rank builds the same model (same seed), takes its slice of a seeded global batch and runs a few
steps with the flat-buffer optimizers (gradient all-reduce through NCCL inside the library); WORLD = 1
runs the whole batch in one process.  The final parameters are written for the parent to compare."""
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

PER_RANK, STEPS = 8, 3


def build(nn):
    np.random.seed(21)
    # no BatchNorm: its per-shard statistics would make the sharded run differ from the one-process run by design
    return nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(8, 12, 3, padding=1), nn.ReLU(),
                         nn.GlobalAvgPool2d(), nn.Flatten(), nn.Linear(12, 5))


def main() -> None:
    rank, world, id_file, out_dir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], Path(sys.argv[4])
    shards = int(sys.argv[5]) if len(sys.argv) > 5 else world          # how many slices make the global batch
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import distributed, nn

    group = distributed.init_from_file(id_file, rank, world, device=rank, timeout_s=120) if world > 1 else None
    rng = np.random.default_rng(77)
    gx = rng.standard_normal((PER_RANK * shards, 3, 16, 16)).astype(np.float32)
    gt = rng.standard_normal((PER_RANK * shards, 5)).astype(np.float32)
    rows = slice(rank * PER_RANK, (rank + 1) * PER_RANK) if world > 1 else slice(None)
    x, t = kd.Tensor.from_numpy(gx[rows]), kd.Tensor.from_numpy(gt[rows])
    res = {}
    for name in ("sgd", "adam"):
        model = build(nn)
        opt = (nn.SGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-3, group=group) if name == "sgd"
               else nn.Adam(model.parameters(), lr=1e-2, weight_decay=1e-3, group=group))
        losses = [nn.train_step(model, opt, x, t).item() for _ in range(STEPS)]
        res[f"{name}/loss"] = np.array(losses, np.float64)
        for i, p in enumerate(model.parameters()):
            res[f"{name}/p{i}"] = p.to_numpy()
    np.savez(out_dir / f"dp_rank{rank}_of{world}.npz", **res)
    if group is not None:
        group.destroy()


if __name__ == "__main__":
    main()
