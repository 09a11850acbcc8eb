"""The reference itself on the host cores: its own CPU Tensor methods, autograd and training step, imported
from the staged copy under ``oracle/_ref/tree`` (see ``oracle/build.py::stage_reference_tree``).
BASELINE INFRASTRUCTURE ONLY: used by the ``cpu_baseline`` legs and the ``--impl reference`` arm of bench.py;
nothing in keydnn_v2_b200 imports it.  Where the staged copy is absent, ``available()`` is False and bench.py
falls back to the NumPy restatement in ``oracle/cpu_baseline.py`` (kind "port").

What runs here is the reference's code, unmodified:
  reductions   ``Tensor.sum(axis)`` / ``Tensor.mean()`` / ``Tensor.max(axis)`` followed by ``backward(grad_out=ones)``
               (src/keydnn/infrastructure/tensor/mixins/reduction/_tensor_sum.py:326-430, _tensor_mean.py:53-81,
               _tensor_max.py:172-269, tensor/_tensor.py:1420-1600)
  CNN step     ``Sequential(...).train_on_batch`` (models/_models.py:402-513) with Conv2d on its OpenMP C++ kernels,
               BatchNorm2d (layers/_batchnorm.py:562-700), MSEFn, SGD (optimizers/_sgd.py:119-140)
The reference has no axis-wise mean and no all-element max (and its SGD has no momentum): those three cases of
the reductions workload are timed as the NumPy expressions of the same form from ``oracle/cpu_baseline.py``, and
the CNN step is timed with the reference's plain SGD.
"""
from __future__ import annotations

import ctypes
import os
import sys
import time
from pathlib import Path
from typing import Dict, Optional

import numpy as np

from . import cpu_baseline

TREE = Path(__file__).resolve().parent / "_ref" / "tree"
_state: Dict[str, object] = {}


def available() -> bool:
    return (TREE / ".staged").exists()


def _import() -> Dict[str, object]:
    """Imports the staged reference package once (CPU paths only; its CUDA library is never opened here)."""
    if _state:
        return _state
    if not available():
        raise RuntimeError("no staged copy of the reference under oracle/_ref/tree")
    if not hasattr(ctypes, "windll"):
        # nine binding modules touch ctypes.windll at import; on the CPU paths none of them resolves a symbol
        class _Kernel32:
            @staticmethod
            def GetProcAddress(handle, name):
                return None

        class _Windll:
            kernel32 = _Kernel32()

        ctypes.windll = _Windll()
    if not hasattr(os, "add_dll_directory"):
        os.add_dll_directory = lambda p: None
    src = str(TREE / "src")
    if src not in sys.path:
        sys.path.insert(0, src)
    from keydnn.domain.device._device import Device
    from keydnn.infrastructure.tensor._tensor import Tensor

    _state.update(Tensor=Tensor, cpu=Device("cpu"))
    return _state


def _tensor(a: np.ndarray, requires_grad: bool = False):
    st = _import()
    t = st["Tensor"](shape=a.shape, device=st["cpu"], requires_grad=requires_grad)
    t.copy_from_numpy(a)
    return t


def reduce_forward_backward(x: np.ndarray, op: str, axis) -> None:
    """One forward + backward (upstream gradient of ones) through the reference's CPU Tensor; the three cases it
    does not have run as the NumPy expressions of the same form."""
    has = (op == "sum") or (op == "mean" and axis is None) or (op == "max" and axis is not None)
    if not has:
        cpu_baseline.reduce_forward_backward(x, op, axis)
        return
    t = _tensor(x, requires_grad=True)
    y = getattr(t, op)() if axis is None else getattr(t, op)(axis=axis)
    if y.shape == ():
        y.backward()
    else:
        y.backward(grad_out=_tensor(np.ones(y.shape, np.float32)))
    assert t.grad is not None and t.grad.shape == x.shape


def time_reduce_workload(x32: np.ndarray, x64: np.ndarray) -> Dict[str, float]:
    """Seconds for one pass over the nine (op, axis) cases on both matrices; same algorithmic byte count as the
    GPU arm (read x forward + write the gradient backward)."""
    t0 = time.perf_counter()
    for x in (x32, x64):
        for op, ax in cpu_baseline.REDUCE_CASES:
            reduce_forward_backward(x, op, ax)
    dt = time.perf_counter() - t0
    return {"seconds": dt, "bytes": float(len(cpu_baseline.REDUCE_CASES) * 2 * (x32.nbytes + x64.nbytes))}


def cnn_training_steps(batch: int, steps: int, warmup: int = 1, seed: int = 1234) -> Dict[str, float]:
    """The benchmark CNN (Conv(3-32)-BN-ReLU-MaxPool2-Conv(32-64)-BN-ReLU-GAP-Flatten-Linear(64-10), MSE, SGD with
    weight decay) trained by the reference on its CPU path for `steps` batches of `batch` samples of (3, 64, 64);
    returns seconds per step and the first / last loss."""
    _import()
    from keydnn.infrastructure._activations import ReLU
    from keydnn.infrastructure._losses import MSEFn
    from keydnn.infrastructure.convolution._conv2d_module import Conv2d
    from keydnn.infrastructure.flatten._flatten_module import Flatten
    from keydnn.infrastructure.fully_connected._linear import Linear
    from keydnn.infrastructure.layers._batchnorm import BatchNorm2d
    from keydnn.infrastructure.models._sequential import Sequential
    from keydnn.infrastructure.optimizers._sgd import SGD
    from keydnn.infrastructure.pooling._pooling_module import GlobalAvgPool2d, MaxPool2d
    from keydnn.infrastructure.tensor._tensor_context import Context

    cpu = _state["cpu"]
    np.random.seed(seed)
    model = Sequential(
        Conv2d(3, 32, 3, padding=1, device=cpu), BatchNorm2d(32, device=cpu), ReLU(), MaxPool2d(2),
        Conv2d(32, 64, 3, padding=1, device=cpu), BatchNorm2d(64, device=cpu), ReLU(), GlobalAvgPool2d(), Flatten(),
        Linear(64, 10, device=cpu, initializer="kaiming"),
    )
    opt = SGD(list(model.parameters()), lr=0.01, weight_decay=1e-4)

    def mse(pred, target):
        ctx = Context(parents=(pred,), backward_fn=lambda g: None)
        loss = MSEFn.forward(ctx, pred, target)
        ctx.backward_fn = lambda g: MSEFn.backward(ctx, g)[:1]
        loss.requires_grad = True
        loss._set_ctx(ctx)
        return loss

    rng = np.random.default_rng(100)
    x = _tensor(rng.standard_normal((batch, 3, 64, 64), dtype=np.float32))
    t = _tensor(np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)])
    losses = []
    for _ in range(warmup):
        losses.append(model.train_on_batch(x, t, loss=mse, optimizer=opt)["loss"])
    t0 = time.perf_counter()
    for _ in range(steps):
        losses.append(model.train_on_batch(x, t, loss=mse, optimizer=opt)["loss"])
    dt = time.perf_counter() - t0
    return {"seconds_per_step": dt / max(1, steps), "loss_first": float(losses[0]), "loss_last": float(losses[-1]),
            "batch": batch, "steps": steps}


def omp_threads() -> Optional[int]:
    """Threads the reference's OpenMP convolution kernels will use (OMP_NUM_THREADS, else all host cores)."""
    v = os.environ.get("OMP_NUM_THREADS")
    try:
        return int(v) if v else os.cpu_count()
    except ValueError:
        return os.cpu_count()
