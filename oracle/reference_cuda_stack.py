"""The reference's own Python stack on its CUDA path, timed over a given native library.  BASELINE INFRASTRUCTURE
ONLY (bench.py --workload dropin runs it twice in child processes: over this repository's drop-in library and over
the reference's own library compiled unmodified, `oracle/_ref/libkeydnn_ref_cuda_full.so`).

What runs is the reference's code from the staged copy under `oracle/_ref/tree`, unmodified: its loader
(native_cuda/python/_native_loader.py:37-150), ctypes bindings, `_CudaStorage`, Tensor dispatch
(tensor/_tensor.py, tensor/mixins/**), autograd (`Tensor.backward`, _tensor.py:1601-1861), pooling Functions
(pooling/_pooling_function.py:62-384), Linear / Sigmoid / SGD.  Only the file at the DLL path differs between the
two runs.  Usage (child process):

    python -m oracle.reference_cuda_stack <path of the library to place, or "ours"> <repeats>

prints one JSON object {workload: milliseconds per iteration}.  Inputs are uploaded once; an iteration is the
forward + backward (or the training step) through the reference's Tensor API, with the device synchronised before
the first and after the last iteration of a loop; the best of three loops is reported.
"""
from __future__ import annotations

import gc
import json
import sys
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
TREE = HERE / "_ref" / "tree"


def main() -> None:
    lib_arg, repeats = sys.argv[1], int(sys.argv[2])
    sys.path.insert(0, str(REPO))
    sys.path.insert(0, str(TREE))
    from keydnn_v2_b200 import dropin

    dropin.install_shim()
    dropin.place(TREE / "src" / "keydnn", lib=None if lib_arg == "ours" else lib_arg)

    from src.keydnn.domain.device._device import Device
    from src.keydnn.infrastructure._activations import Sigmoid
    from src.keydnn.infrastructure.fully_connected._linear import Linear
    from src.keydnn.infrastructure.models._sequential import Sequential
    from src.keydnn.infrastructure.native_cuda.python.maxpool2d_ctypes import cuda_set_device, cuda_synchronize
    from src.keydnn.infrastructure.optimizers._sgd import SGD
    from src.keydnn.infrastructure.pooling._pooling_module import AvgPool2d, GlobalAvgPool2d, MaxPool2d
    from src.keydnn.infrastructure.tensor._tensor import Tensor

    lib = Tensor._get_cuda_lib()
    cuda_set_device(lib, 0)
    cuda = Device("cuda:0")
    rng = np.random.default_rng(0)

    def dev(a, requires_grad=False):
        t = Tensor(shape=a.shape, device=cuda, requires_grad=requires_grad)
        t.copy_from_numpy(a)
        return t

    def timed(fn) -> float:
        # best of three loops: the reference's pooling Contexts reference themselves, so their device buffers wait for
        # the cyclic collector, and a loop in which it happens to run late pays for fresh allocations
        for _ in range(2):
            fn()
        best = float("inf")
        for _ in range(3):
            gc.collect()
            cuda_synchronize(lib)
            t0 = time.perf_counter()
            for _ in range(repeats):
                fn()
            cuda_synchronize(lib)
            best = min(best, (time.perf_counter() - t0) / repeats * 1e3)
        return best

    out = {}
    # element-wise chain with autograd: (a + b) * a / b, negated, summed, backward  (2048 x 2048 fp32)
    a_np = rng.standard_normal((2048, 2048)).astype(np.float32)
    b_np = rng.uniform(0.5, 2.0, (2048, 2048)).astype(np.float32)

    a, b = dev(a_np, True), dev(b_np, True)

    def elementwise():
        a.zero_grad()
        b.zero_grad()
        loss = (-(((a + b) * a) / b)).sum()
        loss.backward()
        return a.grad

    out["elementwise chain + backward, 2048x2048 fp32"] = timed(elementwise)
    # reductions with backward (4096 x 4096 fp32)
    x_np = rng.standard_normal((4096, 4096)).astype(np.float32)
    x, ones = dev(x_np, True), dev(np.ones(4096, np.float32))

    def reductions():
        x.zero_grad()
        x.sum(axis=0).backward(grad_out=ones)
        x.sum(axis=1).backward(grad_out=ones)
        x.max(axis=1).backward(grad_out=ones)
        x.max(axis=0).backward(grad_out=ones)
        x.sum().backward()
        x.mean().backward()
        return x.grad

    out["sum/max axis 0/1, sum, mean + backward, 4096x4096 fp32"] = timed(reductions)
    # pooling Modules forward + backward
    p_np = rng.uniform(-1, 1, (32, 64, 112, 112)).astype(np.float32)
    g_np = rng.standard_normal((32, 64, 56, 56)).astype(np.float32)
    pool = MaxPool2d(kernel_size=2, stride=2)

    px, pg = dev(p_np, True), dev(g_np)

    def maxpool():
        px.zero_grad()
        pool(px).backward(grad_out=pg)
        return px.grad

    out["MaxPool2d(2) fwd+bwd, (32,64,112,112) fp32"] = timed(maxpool)
    q_np = rng.uniform(-1, 1, (64, 256, 56, 56)).astype(np.float32)
    gq_np = rng.standard_normal((64, 256, 28, 28)).astype(np.float32)
    avg = AvgPool2d(kernel_size=3, stride=2, padding=1)

    del px, pg
    qx, qg = dev(q_np, True), dev(gq_np)

    def avgpool():
        qx.zero_grad()
        avg(qx).backward(grad_out=qg)
        return qx.grad

    out["AvgPool2d(3,2,1) fwd+bwd, (64,256,56,56) fp32"] = timed(avgpool)
    r_np = rng.standard_normal((256, 2048, 7, 7)).astype(np.float32)
    gr_np = rng.standard_normal((256, 2048, 1, 1)).astype(np.float32)
    gap = GlobalAvgPool2d()

    del qx, qg
    rx, rg = dev(r_np, True), dev(gr_np)

    def gavgpool():
        rx.zero_grad()
        gap(rx).backward(grad_out=rg)
        return rx.grad

    out["GlobalAvgPool2d fwd+bwd, (256,2048,7,7) fp32"] = timed(gavgpool)
    # a small MLP trained with the reference's SGD on the CUDA path (batch 256, 512-256-10)
    np.random.seed(0)
    model = Sequential(Linear(512, 256, device=cuda), Sigmoid(), Linear(256, 10, device=cuda), Sigmoid())
    opt = SGD(model.parameters(), lr=0.1)
    xb, yb = dev(rng.standard_normal((256, 512)).astype(np.float32)), dev(rng.uniform(0, 1, (256, 10)).astype(np.float32))

    def train_step():
        for p in model.parameters():
            p.zero_grad()
        diff = model(xb) - yb
        loss = (diff * diff).mean()
        loss.backward()
        opt.step()
        return loss

    out["MLP 512-256-10 training step (Linear, Sigmoid, MSE, SGD), batch 256"] = timed(train_step)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
