"""Generate ``tests/golden/ref_cpu_golden.npz`` by RUNNING THE REFERENCE ITSELF.

Run from the repository root, on a machine that has a checkout of the reference
project (its path: first argument, else the KEYDNN_REFERENCE_ROOT environment variable):

    python tests/golden/make_golden.py [REFERENCE_ROOT]

Two sources, both the reference's own code, neither modified:
  * its Python/NumPy CPU path, imported from ``REFERENCE_ROOT/src`` (Tensor ops with
    autograd, pooling Functions, the SGD optimizer);
  * its C++ CPU pooling kernels, compiled by ``oracle/build.py`` from the sources
    where they lie into ``oracle/_ref/libkeydnn_ref_native.so`` and called through
    the C ABI of ``native/src/keydnn_maxpool2d.hpp`` / ``keydnn_avgpool2d.hpp``.

The fixtures are small seeded cases; the test-suite compares both the CPU oracle
(``oracle/``) and the CUDA library against them.  The generated file is committed;
the reference is not needed to run the tests.
"""
from __future__ import annotations

import ctypes
import sys
import warnings
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
from oracle.build import DEFAULT_REF_ROOT  # noqa: E402

REF_ROOT = Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_REF_ROOT
sys.dont_write_bytecode = True
sys.path.insert(0, str(REF_ROOT / "src"))
sys.path.insert(0, str(REPO))
warnings.simplefilter("ignore")

# The reference's CUDA binding modules resolve symbols through ctypes.windll at import time (they are
# imported even on the CPU path of Conv2d); give them a stand-in so the CPU path can be imported here.
import os  # noqa: E402

if not hasattr(ctypes, "windll"):
    class _Kernel32:
        @staticmethod
        def GetProcAddress(handle, name):
            return None

    class _Windll:
        kernel32 = _Kernel32()

    ctypes.windll = _Windll()
if not hasattr(os, "add_dll_directory"):
    os.add_dll_directory = lambda p: None

from keydnn.domain.device._device import Device  # noqa: E402
from keydnn.infrastructure.optimizers._sgd import SGD  # noqa: E402
from keydnn.infrastructure._parameter import Parameter  # noqa: E402
from keydnn.infrastructure.pooling._pooling_function import (  # noqa: E402
    AvgPool2dFn,
    GlobalAvgPool2dFn,
    MaxPool2dFn,
)
from keydnn.infrastructure.tensor._tensor import Tensor  # noqa: E402
from keydnn.infrastructure.tensor._tensor_context import Context  # noqa: E402

from oracle import build as oracle_build  # noqa: E402

CPU = Device("cpu")
OUT: dict[str, np.ndarray] = {}


def tensor(a: np.ndarray, requires_grad: bool = False) -> Tensor:
    t = Tensor(shape=a.shape, device=CPU, requires_grad=requires_grad)
    t.copy_from_numpy(a)
    return t


def put(name: str, a) -> None:
    OUT[name] = np.array(a, copy=True, order="C")      # a copy: some to_numpy() results alias live buffers


# ---------------------------------------------------------------------------
# pooling through the reference Functions (NumPy loops on this path)
# ---------------------------------------------------------------------------
POOL_CASES = [
    # name, shape, kernel, stride, padding
    ("k2s2p0", (2, 3, 8, 8), 2, 2, 0),
    ("k3s2p1", (2, 2, 8, 8), 3, 2, 1),
    ("k3s1p1", (1, 2, 7, 5), 3, 1, 1),
    ("k2s2p0_odd", (1, 2, 7, 9), 2, 2, 0),
    ("k23s21p10", (1, 1, 9, 10), (2, 3), (2, 1), (1, 0)),
]


def pool_cases() -> None:
    rng = np.random.default_rng(1)
    for name, shape, k, s, p in POOL_CASES:
        x = rng.uniform(-1, 1, shape).astype(np.float32)
        put(f"pool/{name}/x", x)
        for kind, Fn in (("max", MaxPool2dFn), ("avg", AvgPool2dFn)):
            xt = tensor(x, True)
            ctx = Context(parents=(xt,), backward_fn=lambda g: None)
            y = Fn.forward(ctx, xt, kernel_size=k, stride=s, padding=p)
            yn = y.to_numpy()
            go = rng.standard_normal(yn.shape).astype(np.float32)
            (gx,) = Fn.backward(ctx, tensor(go))
            put(f"pool/{name}/{kind}_y", yn)
            put(f"pool/{name}/{kind}_go", go)
            put(f"pool/{name}/{kind}_gx", gx.to_numpy())
            if kind == "max":
                put(f"pool/{name}/max_idx", np.asarray(ctx.saved_meta["argmax_idx"], dtype=np.int64))
    # tie-heavy input: first index must win (tests/infrastructure/pool2d/test_pool2d_tie_breaking.py)
    x = (np.round(rng.uniform(-1, 1, (1, 2, 6, 6)) * 2) / 2).astype(np.float32)
    put("pool/ties/x", x)
    xt = tensor(x, True)
    ctx = Context(parents=(xt,), backward_fn=lambda g: None)
    y = MaxPool2dFn.forward(ctx, xt, kernel_size=2, stride=2, padding=0)
    go = np.ones(y.shape, np.float32)
    (gx,) = MaxPool2dFn.backward(ctx, tensor(go))
    put("pool/ties/max_y", y.to_numpy())
    put("pool/ties/max_idx", np.asarray(ctx.saved_meta["argmax_idx"], dtype=np.int64))
    put("pool/ties/max_gx", gx.to_numpy())
    # global average pool
    x = rng.standard_normal((3, 5, 7, 7)).astype(np.float32)
    xt = tensor(x, True)
    ctx = Context(parents=(xt,), backward_fn=lambda g: None)
    y = GlobalAvgPool2dFn.forward(ctx, xt)
    go = rng.standard_normal(y.shape).astype(np.float32)
    (gx,) = GlobalAvgPool2dFn.backward(ctx, tensor(go))
    put("gap/x", x)
    put("gap/y", y.to_numpy())
    put("gap/go", go)
    put("gap/gx", gx.to_numpy())


# ---------------------------------------------------------------------------
# pooling through the reference's C++ kernels (padded-plane C ABI)
# ---------------------------------------------------------------------------
def native_pool_cases() -> None:
    libs = oracle_build.build_reference(REF_ROOT)
    lib = ctypes.CDLL(str(libs["native"]))
    rng = np.random.default_rng(2)
    P = lambda a: ctypes.c_void_p(a.ctypes.data)  # noqa: E731
    for tag, dt in (("f32", np.float32), ("f64", np.float64)):
        N, C, H, W, k, s, p = 2, 3, 9, 10, 3, 2, 1
        x = rng.uniform(-1, 1, (N, C, H, W)).astype(dt)
        Hp, Wp = H + 2 * p, W + 2 * p
        Ho, Wo = (Hp - k) // s + 1, (Wp - k) // s + 1
        for kind, padv in (("max", -np.inf), ("avg", 0.0)):
            xp = np.pad(x, ((0, 0), (0, 0), (p, p), (p, p)), constant_values=dt(padv))
            xp = np.ascontiguousarray(xp)
            y = np.zeros((N, C, Ho, Wo), dt)
            go = rng.standard_normal((N, C, Ho, Wo)).astype(dt)
            gxp = np.zeros((N, C, Hp, Wp), dt)
            if kind == "max":
                idx = np.zeros((N, C, Ho, Wo), np.int64)
                getattr(lib, f"keydnn_maxpool2d_forward_{tag}")(P(xp), P(y), P(idx), N, C, Hp, Wp, Ho, Wo, k, k, s, s)
                getattr(lib, f"keydnn_maxpool2d_backward_{tag}")(P(go), P(idx), P(gxp), N, C, Ho, Wo, Hp, Wp)
                put(f"native/{tag}/max_idx", idx)
            else:
                getattr(lib, f"keydnn_avgpool2d_forward_{tag}")(P(xp), P(y), N, C, Hp, Wp, Ho, Wo, k, k, s, s)
                getattr(lib, f"keydnn_avgpool2d_backward_{tag}")(P(go), P(gxp), N, C, Ho, Wo, Hp, Wp, k, k, s, s)
            put(f"native/{tag}/{kind}_y", y)
            put(f"native/{tag}/{kind}_go", go)
            put(f"native/{tag}/{kind}_gx", gxp[:, :, p:p + H, p:p + W])
        put(f"native/{tag}/x", x)
    put("native/geom", np.array([2, 3, 9, 10, 3, 2, 1], np.int64))


# ---------------------------------------------------------------------------
# Tensor ops with autograd on the reference CPU path
# ---------------------------------------------------------------------------
def tensor_cases() -> None:
    rng = np.random.default_rng(3)
    a = rng.standard_normal((6, 10)).astype(np.float32)
    b = rng.uniform(0.5, 2.0, (6, 10)).astype(np.float32)
    g = rng.standard_normal((6, 10)).astype(np.float32)
    put("ew/a", a)
    put("ew/b", b)
    put("ew/g", g)
    ops = {"add": lambda x, y: x + y, "sub": lambda x, y: x - y, "mul": lambda x, y: x * y, "div": lambda x, y: x / y}
    for name, fn in ops.items():
        ta, tb = tensor(a, True), tensor(b, True)
        y = fn(ta, tb)
        y.backward(tensor(g))
        put(f"ew/{name}_y", y.to_numpy())
        put(f"ew/{name}_ga", ta.grad.to_numpy())
        put(f"ew/{name}_gb", tb.grad.to_numpy())
    ta = tensor(a, True)
    y = -ta
    y.backward(tensor(g))
    put("ew/neg_y", y.to_numpy())
    put("ew/neg_ga", ta.grad.to_numpy())
    cmps = {"gt": lambda x, y: x > y, "ge": lambda x, y: x >= y, "lt": lambda x, y: x < y, "le": lambda x, y: x <= y}
    a2 = np.round(a * 2) / 2
    b2 = np.round(b * 2) / 2
    put("ew/a2", a2.astype(np.float32))
    put("ew/b2", b2.astype(np.float32))
    for name, fn in cmps.items():
        put(f"ew/{name}_y", fn(tensor(a2.astype(np.float32)), tensor(b2.astype(np.float32))).to_numpy())
    put("ew/gt_scalar_y", (tensor(a) > 0.0).to_numpy())
    put("ew/add_scalar_y", (tensor(a) + 1.5).to_numpy())
    put("ew/mul_scalar_y", (tensor(a) * 0.3).to_numpy())
    put("ew/div_scalar_y", (tensor(a) / 0.7).to_numpy())
    put("ew/sub_scalar_y", (tensor(a) - 0.25).to_numpy())

    # reductions
    x = rng.standard_normal((7, 12)).astype(np.float32)
    put("red/x", x)
    tx = tensor(x, True)
    y = tx.sum()
    y.backward()
    put("red/sum_all_y", y.to_numpy())
    put("red/sum_all_gx", tx.grad.to_numpy())
    tx = tensor(x, True)
    y = tx.mean()
    y.backward()
    put("red/mean_all_y", y.to_numpy())
    put("red/mean_all_gx", tx.grad.to_numpy())
    for axis in (0, 1):
        tx = tensor(x, True)
        y = tx.sum(axis=axis)
        go = rng.standard_normal(y.shape).astype(np.float32)
        y.backward(tensor(go))
        put(f"red/sum_axis{axis}_y", y.to_numpy())
        put(f"red/sum_axis{axis}_go", go)
        put(f"red/sum_axis{axis}_gx", tx.grad.to_numpy())
        tx = tensor(x, True)
        y = tx.max(axis=axis)
        go = rng.standard_normal(y.shape).astype(np.float32)
        y.backward(tensor(go))
        put(f"red/max_axis{axis}_y", y.to_numpy())
        put(f"red/max_axis{axis}_go", go)
        put(f"red/max_axis{axis}_gx", tx.grad.to_numpy())

    # SGD with coupled weight decay, two steps (optimizers/_sgd.py:119-140)
    p0 = rng.standard_normal(37).astype(np.float32)
    g1 = (rng.standard_normal(37) * 1e-2).astype(np.float32)
    g2 = (rng.standard_normal(37) * 1e-2).astype(np.float32)
    par = Parameter(shape=p0.shape, device=CPU, requires_grad=True)
    par.copy_from_numpy(p0)
    opt = SGD([par], lr=0.01, weight_decay=1e-4)
    steps = []
    for gi in (g1, g2):
        par.zero_grad()
        par._set_grad(tensor(gi)) if hasattr(par, "_set_grad") else setattr(par, "_grad", tensor(gi))
        opt.step()
        steps.append(par.to_numpy().copy())
    put("sgd/p0", p0)
    put("sgd/g1", g1)
    put("sgd/g2", g2)
    put("sgd/p1", steps[0])
    put("sgd/p2", steps[1])


def cnn_case() -> None:
    """One training step of a scaled-down copy of the benchmark CNN on the reference's CPU path:
    Conv(3->4,3x3,p1)-BN-ReLU-MaxPool(2)-Conv(4->6,3x3,p1)-BN-ReLU-GlobalAvgPool-Flatten-Linear(6->3), MSE, SGD."""
    from keydnn.infrastructure._activations import ReLU
    from keydnn.infrastructure._losses import MSEFn
    from keydnn.infrastructure.convolution._conv2d_module import Conv2d
    from keydnn.infrastructure.flatten._flatten_module import Flatten
    from keydnn.infrastructure.fully_connected._linear import Linear
    from keydnn.infrastructure.layers._batchnorm import BatchNorm2d
    from keydnn.infrastructure.models._sequential import Sequential
    from keydnn.infrastructure.pooling._pooling_module import GlobalAvgPool2d, MaxPool2d

    np.random.seed(5)
    model = Sequential(
        Conv2d(3, 4, 3, padding=1, device=CPU), BatchNorm2d(4, device=CPU), ReLU(), MaxPool2d(2),
        Conv2d(4, 6, 3, padding=1, device=CPU), BatchNorm2d(6, device=CPU), ReLU(), GlobalAvgPool2d(), Flatten(),
        Linear(6, 3, device=CPU, initializer="kaiming"),
    )
    params = list(model.parameters())
    for i, p in enumerate(params):
        put(f"cnn/p{i}_init", p.to_numpy())
    rng = np.random.default_rng(9)
    x = rng.standard_normal((4, 3, 8, 8)).astype(np.float32)
    t = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 4)]
    put("cnn/x", x)
    put("cnn/t", t)
    pred = model(tensor(x))
    ctx = Context(parents=(pred,), backward_fn=lambda g: None)
    tt = tensor(t)
    loss = MSEFn.forward(ctx, pred, tt)
    ctx.backward_fn = lambda g: MSEFn.backward(ctx, g)[:1]
    loss.requires_grad = True
    loss._set_ctx(ctx)
    loss.backward()
    put("cnn/pred", pred.to_numpy())
    put("cnn/loss", loss.to_numpy())
    for i, p in enumerate(params):
        put(f"cnn/p{i}_grad", p.grad.to_numpy())
    SGD(params, lr=0.01, weight_decay=1e-4).step()
    for i, p in enumerate(params):
        put(f"cnn/p{i}_after", p.to_numpy())
    put("cnn/n_params", np.array([len(params)], np.int64))


def _run_fn(fn, arrays, go, **kw):
    """forward + backward of a reference Function on its CPU path; returns (y, grads of the inputs that get one)."""
    ts = [tensor(a) for a in arrays]
    ctx = Context(parents=tuple(ts), backward_fn=lambda g: None)
    y = fn.forward(ctx, *ts, **kw)
    g = fn.backward(ctx, tensor(go))
    if not isinstance(g, (tuple, list)):
        g = (g,)
    return y.to_numpy(), [None if t is None else t.to_numpy() for t in g]


def activation_cases() -> None:
    """Activations (_function.py), unary ops, losses (_losses.py) and Adam (optimizers/_adam.py) on the CPU path."""
    from keydnn.infrastructure._function import ExpFn, LeakyReLUFn, ReLUFn, SigmoidFn, SoftmaxFn, TanhFn
    from keydnn.infrastructure._losses import BinaryCrossEntropyFn, CategoricalCrossEntropyFn, MSEFn, SSEFn
    from keydnn.infrastructure.optimizers._adam import Adam

    rng = np.random.default_rng(31)
    x = (rng.standard_normal((13, 37)) * 2.0).astype(np.float32)
    x.flat[:4] = [0.0, -0.0, 1e-3, -1e-3]
    go = rng.standard_normal(x.shape).astype(np.float32)
    put("act/x", x)
    put("act/go", go)
    for name, fn, kw in (("exp", ExpFn, {}), ("sigmoid", SigmoidFn, {}), ("relu", ReLUFn, {}), ("tanh", TanhFn, {}),
                         ("leaky", LeakyReLUFn, {"alpha": 0.1}), ("softmax1", SoftmaxFn, {"axis": -1}),
                         ("softmax0", SoftmaxFn, {"axis": 0})):
        y, g = _run_fn(fn, [x], go, **kw)
        put(f"act/{name}_y", y)
        put(f"act/{name}_gx", g[0])
    xp = rng.uniform(0.05, 4.0, x.shape).astype(np.float32)
    put("act/xpos", xp)
    for name in ("log", "sqrt"):
        t = tensor(xp, True)
        y = getattr(t, name)()
        y.backward(tensor(go))
        put(f"act/{name}_y", y.to_numpy())
        put(f"act/{name}_gx", t.grad.to_numpy())

    pred = rng.uniform(0.05, 0.95, (16, 10)).astype(np.float32)
    pred /= pred.sum(1, keepdims=True)
    onehot = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 16)]
    binary = (rng.uniform(size=pred.shape) > 0.5).astype(np.float32)
    target = rng.standard_normal(pred.shape).astype(np.float32)
    g_up = np.array(0.7, np.float32)                                   # upstream gradient of the scalar loss
    put("loss/pred", pred)
    put("loss/onehot", onehot)
    put("loss/binary", binary)
    put("loss/target", target)
    put("loss/g", g_up)
    for name, fn, tgt in (("sse", SSEFn, target), ("mse", MSEFn, target), ("bce", BinaryCrossEntropyFn, binary),
                          ("cce", CategoricalCrossEntropyFn, onehot)):
        y, g = _run_fn(fn, [pred, tgt], g_up)
        put(f"loss/{name}_y", y)
        put(f"loss/{name}_gpred", g[0])
        if g[1] is not None:
            put(f"loss/{name}_gtarget", g[1])

    # Adam with coupled weight decay, three steps
    p0 = rng.standard_normal(53).astype(np.float32)
    grads = [(rng.standard_normal(53) * 1e-1).astype(np.float32) for _ in range(3)]
    for tag, wd in (("adam", 0.0), ("adam_wd", 1e-2)):
        par = Parameter(shape=p0.shape, device=CPU, requires_grad=True)
        par.copy_from_numpy(p0)
        opt = Adam([par], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd)
        for k, gi in enumerate(grads):
            par.zero_grad()
            par._set_grad(tensor(gi)) if hasattr(par, "_set_grad") else setattr(par, "_grad", tensor(gi))
            opt.step()
            put(f"{tag}/p{k + 1}", par.to_numpy())
        st = next(iter(opt._state.values()))
        put(f"{tag}/m3", st["m"].to_numpy())
        put(f"{tag}/v3", st["v"].to_numpy())
    put("adam/p0", p0)
    for k, gi in enumerate(grads):
        put(f"adam/g{k + 1}", gi)


def main() -> None:
    cnn_case()
    pool_cases()
    native_pool_cases()
    tensor_cases()
    activation_cases()
    out = REPO / "tests" / "golden" / "ref_cpu_golden.npz"
    np.savez_compressed(out, **OUT)
    print(f"wrote {out} ({out.stat().st_size} bytes, {len(OUT)} arrays)")


if __name__ == "__main__":
    main()
