"""The reference's CPU path for the benchmark workloads, restated as the NumPy expressions it
runs.  TEST / BASELINE INFRASTRUCTURE ONLY (the `cpu_baseline` leg and `--impl reference` arm of
bench.py); nothing in keydnn_v2_b200 imports it.

The reference computes reductions and elementwise ops on the CPU with single-threaded NumPy
calls inside its Tensor methods (paths below are under src/keydnn/infrastructure/):
  sum   forward  np.sum(x[, axis])                          tensor/mixins/reduction/_tensor_sum.py:372-385
        backward np.ones(shape, f32) * g                    _tensor_sum.py:389-419
  mean  forward  np.sum(x) / n                              _tensor_mean.py:53-54
        backward np.ones(shape, f32) * (g / n)              _tensor_mean.py:78-81
  max   forward  np.max(x, axis)                            _tensor_max.py:221
        backward (x == m) * g                               _tensor_max.py:257-258
  add/sub/mul/div  a op b                                   tensor/mixins/arithmetic/_tensor_addition.py:158 etc.
and pooling with its C++ kernels (native/src/keydnn_{max,avg}pool2d.cpp), which oracle/build.py
compiles unmodified into oracle/_ref/libkeydnn_ref_native.so.
Axis-wise mean and all-element max do not exist in the reference; they are timed as the NumPy
expressions of the same form (np.sum(x, axis) / extent; np.max(x) with an equality mask).
"""
from __future__ import annotations

import time
from typing import Dict, List, Tuple

import numpy as np

REDUCE_CASES: List[Tuple[str, object]] = [(op, ax) for op in ("sum", "mean", "max") for ax in (0, 1, None)]


def reduce_forward_backward(x: np.ndarray, op: str, axis) -> Tuple[np.ndarray, np.ndarray]:
    """One forward + backward (upstream gradient of ones) exactly as the CPU Tensor methods do it."""
    if op == "sum":
        y = np.sum(x) if axis is None else np.sum(x, axis=axis)
        g = np.ones(np.shape(y), x.dtype)
        gx = np.ones(x.shape, x.dtype) * (g if axis is None else np.expand_dims(g, axis))
    elif op == "mean":
        n = x.size if axis is None else x.shape[axis]
        y = (np.sum(x) if axis is None else np.sum(x, axis=axis)) / n
        g = np.ones(np.shape(y), x.dtype)
        gx = np.ones(x.shape, x.dtype) * ((g if axis is None else np.expand_dims(g, axis)) / n)
    else:
        y = np.max(x) if axis is None else np.max(x, axis=axis)
        g = np.ones(np.shape(y), x.dtype)
        m = y if axis is None else np.expand_dims(y, axis)
        gx = (x == m).astype(x.dtype) * (g if axis is None else np.expand_dims(g, axis))
    return np.asarray(y), gx


def time_reduce_workload(x32: np.ndarray, x64: np.ndarray, repeats: int = 1) -> Dict[str, float]:
    """Seconds for one pass over all (op, axis) cases on both matrices; bytes use the same
    algorithmic count as the GPU arm (read x forward + write grad backward)."""
    t0 = time.perf_counter()
    for _ in range(repeats):
        for x in (x32, x64):
            for op, ax in REDUCE_CASES:
                reduce_forward_backward(x, op, ax)
    dt = (time.perf_counter() - t0) / repeats
    nbytes = len(REDUCE_CASES) * 2 * (x32.nbytes + x64.nbytes)
    return {"seconds": dt, "bytes": float(nbytes)}
