"""Row-sharded reductions on 2+ GPUs of one box: one process per GPU, NCCL inside the library.
Skipped on a single-GPU box (the 1-GPU path of the same code is covered by bench.py and smoke)."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def _device_count() -> int:
    import ctypes

    from keydnn_v2_b200 import load

    n = ctypes.c_int(0)
    load().call("keydnn_cuda_device_count", ctypes.byref(n))
    return n.value


def test_sharded_reductions_match_numpy_on_the_whole_matrix(tmp_path):
    world = min(_device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(HERE / "_sharded_worker.py"), str(r), str(world),
                               str(tmp_path / "nccl_id"), str(tmp_path)], env=env) for r in range(world)]
    try:
        codes = [p.wait(timeout=300) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert codes == [0] * world
    res = [dict(np.load(tmp_path / f"rank{r}.npz")) for r in range(world)]
    for tag, dt, R, C in (("f32", np.float32, 96, 520), ("f64", np.float64, 40, 264)):
        full = np.random.default_rng(5).standard_normal((R * world, C))
        full = (np.round(full * 4) / 4).astype(dt)
        full[3, 7] = full[R * world - 2, 7] = 9.0
        tol = dict(rtol=1e-5, atol=1e-5) if dt == np.float32 else dict(rtol=1e-12, atol=1e-12)
        f64 = full.astype(np.float64)
        for ax in (0, 1, None):
            for r in range(world):
                rows = slice(r * R, (r + 1) * R)
                ys, ym, yx = (res[r][f"{tag}/{op}/{ax}/y"] for op in ("sum", "mean", "max"))
                gs, gm, gxm = (res[r][f"{tag}/{op}/{ax}/gx"] for op in ("sum", "mean", "max"))
                # the bucketed exchange (one all-reduce + one all-gather for everything) gives the same bits
                for op in ("sum", "mean", "max"):
                    for what in ("y", "gx"):
                        np.testing.assert_array_equal(res[r][f"{tag}/bucket/{op}/{ax}/{what}"], res[r][f"{tag}/{op}/{ax}/{what}"],
                                                      err_msg=f"bucket {tag} {op} {ax} {what}")
                        # one shared bucket for both matrices (a single all-gather, sums formed locally in rank
                        # order): the inputs are multiples of 1/4, so every order of addition gives the same bits
                        np.testing.assert_array_equal(res[r][f"{tag}/shared/{op}/{ax}/{what}"], res[r][f"{tag}/{op}/{ax}/{what}"],
                                                      err_msg=f"shared bucket {tag} {op} {ax} {what}")
                if ax == 0:
                    np.testing.assert_array_equal(res[r][f"{tag}/partial/mean/0/y"], ym)
                    np.testing.assert_array_equal(res[r][f"{tag}/partial/sum/0/y"], ys)     # untouched by the partial bucket
                if ax is None:
                    np.testing.assert_array_equal(res[r][f"{tag}/partial/max/None/y"], yx)
                if ax == 1:
                    np.testing.assert_allclose(ys, f64[rows].sum(1), **tol)
                    np.testing.assert_allclose(ym, f64[rows].mean(1), **tol)
                    np.testing.assert_array_equal(yx, full[rows].max(1))
                    want = np.zeros((R, C), dt)
                    want[np.arange(R), full[rows].argmax(1)] = 1
                    np.testing.assert_array_equal(gxm, want)
                    np.testing.assert_allclose(gm, np.full((R, C), 1.0 / C), **tol)
                else:
                    axis = 0 if ax == 0 else None
                    np.testing.assert_allclose(ys, np.atleast_1d(f64.sum(axis)), **tol)
                    np.testing.assert_allclose(ym, np.atleast_1d(f64.mean(axis)), **tol)
                    np.testing.assert_array_equal(yx, np.atleast_1d(full.max(axis)))
                    want = np.zeros_like(full)
                    if ax == 0:
                        want[full.argmax(0), np.arange(C)] = 1       # first (lowest-rank) maximum only
                        n = R * world
                    else:
                        want.reshape(-1)[full.argmax()] = 1
                        n = full.size
                    np.testing.assert_array_equal(gxm, want[rows])
                    np.testing.assert_allclose(gm, np.full((R, C), 1.0 / n), **tol)
                np.testing.assert_array_equal(gs, np.ones((R, C), dt))


def test_data_parallel_steps_equal_one_process_on_the_whole_batch(tmp_path):
    """SGD-momentum and Adam over the flat gradient buffer with an NCCL all-reduce: after three steps every
    rank holds the same parameters, and they equal a one-process run on the concatenated batch (the mean
    loss makes the averaged shard gradients the full-batch gradient)."""
    world = min(_device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    worker = str(HERE / "_dp_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), str(world), str(tmp_path / "nccl_id_dp"), str(tmp_path)], env=env)
             for r in range(world)]
    try:
        codes = [p.wait(timeout=300) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert codes == [0] * world
    one = subprocess.run([sys.executable, worker, "0", "1", str(tmp_path / "unused"), str(tmp_path), str(world)], env=env, timeout=300)
    assert one.returncode == 0
    whole = dict(np.load(tmp_path / "dp_rank0_of1.npz"))
    ranks = [dict(np.load(tmp_path / f"dp_rank{r}_of{world}.npz")) for r in range(world)]
    for key in whole:
        if key.endswith("/loss"):
            # each rank reports the loss of its own slice; their mean is the whole-batch loss
            np.testing.assert_allclose(np.mean([r[key] for r in ranks], axis=0), whole[key], rtol=1e-4)
            continue
        for r in ranks[1:]:
            np.testing.assert_array_equal(r[key], ranks[0][key], err_msg=key)       # replicas stay identical
        np.testing.assert_allclose(ranks[0][key], whole[key], rtol=2e-3, atol=2e-5, err_msg=key)
