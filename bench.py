"""Benchmark of the reduction hot path (configuration [1] of the benchmark definition) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--kernels all|none]

A step is one pass of sum / mean / max over axis 0, axis 1 and all axes, each followed by its
backward with an upstream gradient of ones, on an fp32 (8192, 8192) and an fp64 (4096, 4096)
matrix per GPU (rows sharded across ranks; partials of axis-0 and all-axes reductions cross
NVLink through NCCL).  `value` is algorithmic bytes moved per second by all ranks, inputs
resident in HBM; `e2e` is the same through the Tensor API with pinned host inputs copied in and
results copied out every step.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import ctypes
import gc
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

ROWS32, COLS32 = 8192, 8192
ROWS64, COLS64 = 4096, 4096
OPS = [(op, ax) for op in ("sum", "mean", "max") for ax in (0, 1, None)]
METRIC = "fwd+bwd HBM GB/s (sum/mean/max reductions over axis 0, axis 1, all axes; fp32 8192^2 + fp64 4096^2)"


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch of each kernel of the step, from one
# `ncu --set full` capture at these sizes (summary committed under profiles/).  Writes are under-counted there:
# lines still dirty in L2 when a kernel ends are not in its DRAM count.
NCU_TRAFFIC_BYTES = {
    "sum_axis0_fwd_f32": 272715000,
    "sum_axis0_fwd_f64": 137865000,
    "sum_axis0_bwd_f32": 209817000,
    "sum_axis0_bwd_f64": 75364000,
    "sum_axis1_fwd_f32": 272213000,
    "sum_axis1_fwd_f64": 137958000,
    "sum_axis1_bwd_f32": 211139000,
    "sum_axis1_bwd_f64": 77029000,
    "sum_all_fwd_f32": 273015000,
    "sum_all_fwd_f64": 140446000,
    "sum_all_bwd_f32": 210100000,
    "sum_all_bwd_f64": 74301000,
    "mean_axis0_fwd_f32": 271950000,
    "mean_axis0_fwd_f64": 138020000,
    "mean_axis0_bwd_f32": 209788000,
    "mean_axis0_bwd_f64": 75297000,
    "mean_axis1_fwd_f32": 272030000,
    "mean_axis1_fwd_f64": 137968000,
    "mean_axis1_bwd_f32": 212215000,
    "mean_axis1_bwd_f64": 76049000,
    "mean_all_fwd_f32": 271924000,
    "mean_all_fwd_f64": 137805000,
    "mean_all_bwd_f32": 209136000,
    "mean_all_bwd_f64": 75153000,
    "max_axis0_fwd_f32": 275074000,
    "max_axis0_fwd_f64": 139061000,
    "max_axis0_bwd_f32": 209138000,
    "max_axis0_bwd_f64": 76473000,
    "max_axis1_fwd_f32": 271911000,
    "max_axis1_fwd_f64": 138318000,
    "max_axis1_bwd_f32": 209431000,
    "max_axis1_bwd_f64": 75042000,
    "max_all_fwd_f32": 271762000,
    "max_all_fwd_f64": 138227000,
    "max_all_bwd_f32": 209150000,
    "max_all_bwd_f64": 74351000,
}


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def measured_peak_gbs() -> tuple[float, str]:
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------
# clocks sampled during the timed region
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.first = 0

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def mark(self) -> None:
        """Samples from here on are the ones reported (all of them if none arrives afterwards)."""
        self.first = len(self.lines)

    def _pump(self) -> None:
        assert self.proc and self.proc.stdout
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in (self.lines[self.first:] or self.lines):
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# device-side timing with the library's own events (its launches are on its own stream)
# ---------------------------------------------------------------------------
class Timer:
    def __init__(self, lib) -> None:
        self.lib = lib
        a, b = ctypes.c_uint64(0), ctypes.c_uint64(0)
        lib.call("keydnn_cuda_event_create", ctypes.byref(a))
        lib.call("keydnn_cuda_event_create", ctypes.byref(b))
        self.a, self.b = a.value, b.value

    def start(self) -> None:
        self.lib.call("keydnn_cuda_event_record", self.a)

    def stop_ms(self) -> float:
        self.lib.call("keydnn_cuda_event_record", self.b)
        self.lib.call("keydnn_cuda_event_synchronize", self.b)
        ms = ctypes.c_float(0)
        self.lib.call("keydnn_cuda_event_elapsed_ms", self.a, self.b, ctypes.byref(ms))
        return float(ms.value)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def algorithmic_bytes_per_step() -> float:
    """Forward reads the matrix, backward writes the gradient (outputs <= 96 KB are ignored)."""
    per_matrix = ROWS32 * COLS32 * 4 + ROWS64 * COLS64 * 8
    return float(len(OPS) * 2 * per_matrix)


def kernel_table(lib, reducers, timer, reps: int, peak: float) -> list[dict]:
    """Average device time of each forward and backward kernel, `reps` launches back to back."""
    rows = []
    for red, tag in reducers:
        nbytes = red.x.nbytes
        for op, ax in OPS:
            for phase in ("fwd", "bwd"):
                red.forward(op, ax)
                fn = (lambda: red.forward(op, ax)) if phase == "fwd" else (lambda: red.backward(op, ax))
                for _ in range(3):
                    fn()
                timer.start()
                for _ in range(reps):
                    fn()
                ms = timer.stop_ms() / reps
                gbs = nbytes / ms / 1e6
                rows.append({"kernel": f"{op}_{'all' if ax is None else 'axis%d' % ax}_{phase}_{tag}", "us": round(ms * 1e3, 2),
                             "gbs": round(gbs, 1), "frac": round(gbs / peak, 4), "bytes": nbytes})
    return rows


def suite_table(lib, timer, peak: float, reps: int = 10, warm: int = 3) -> list[dict]:
    """Per-kernel device time for the other benchmark configurations (pool, elementwise,
    optimizer step), each launched `reps` times back to back on inputs larger than L2."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import pooling

    T = kd.Tensor
    rng = np.random.default_rng(7)
    rows: list[dict] = []

    def timed(name: str, nbytes: float, fn) -> None:
        for _ in range(warm):
            fn()
        timer.start()
        for _ in range(reps):
            fn()
        ms = timer.stop_ms() / reps
        gbs = nbytes / ms / 1e6
        rows.append({"kernel": name, "us": round(ms * 1e3, 2), "gbs": round(gbs, 1), "frac": round(gbs / peak, 4),
                     "bytes": int(nbytes)})

    def rand(shape, lo=None):
        a = rng.standard_normal(shape, dtype=np.float32) if lo is None else rng.uniform(lo[0], lo[1], shape).astype(np.float32)
        return T.from_numpy(a)

    # configs[0]: MaxPool2d k2 s2 p0 on (32,64,112,112)
    x = rand((32, 64, 112, 112), (-1, 1))
    go = rand((32, 64, 56, 56))
    y, idx = pooling.maxpool2d_forward(x, kernel_size=2, stride=2, padding=0)
    gx = T.empty(x.shape)
    nb = x.nbytes + y.nbytes + y.numel * 8
    timed("maxpool2d_fwd_c1_f32", nb, lambda: lib.call("keydnn_cuda_maxpool2d_forward_ex_f32", x.data, y.data, idx.dev_ptr,
                                                      32, 64, 112, 112, 56, 56, 2, 2, 2, 2, 0, 0))
    timed("maxpool2d_bwd_c1_f32", nb, lambda: lib.call("keydnn_cuda_maxpool2d_backward_ex_f32", go.data, idx.dev_ptr, gx.data,
                                                      32, 64, 112, 112, 56, 56, 2, 2, 2, 2, 0, 0))
    del x, go, y, idx, gx
    # configs[3]: AvgPool2d k3 s2 p1 on (256,256,56,56); GlobalAvgPool on (256,2048,7,7)
    x = rand((256, 256, 56, 56), (-1, 1))
    y = T.empty((256, 256, 28, 28))
    gx = T.empty(x.shape)
    nb = x.nbytes + y.nbytes
    timed("avgpool2d_fwd_c4_f32", nb, lambda: lib.call("keydnn_cuda_avgpool2d_forward_ex_f32", x.data, y.data, 256, 256, 56, 56,
                                                      28, 28, 3, 3, 2, 2, 1, 1))
    timed("avgpool2d_bwd_c4_f32", nb, lambda: lib.call("keydnn_cuda_avgpool2d_backward_ex_f32", y.data, gx.data, 256, 256, 56,
                                                      56, 28, 28, 3, 3, 2, 2, 1, 1))
    del x, y, gx
    x = rand((256, 2048, 7, 7))
    y = T.empty((256, 2048, 1, 1))
    gx = T.empty(x.shape)
    nb = x.nbytes + y.nbytes
    timed("global_avgpool_fwd_c4_f32", nb, lambda: lib.call("keydnn_cuda_global_avgpool2d_forward_f32", x.data, y.data, 256, 2048, 7, 7))
    timed("global_avgpool_bwd_c4_f32", nb, lambda: lib.call("keydnn_cuda_global_avgpool2d_backward_f32", y.data, gx.data, 256, 2048, 7, 7))
    del x, y, gx
    # configs[2]: elementwise on 2^28 fp32 elements, SGD-momentum on 25,165,824
    n = 1 << 28
    a = T.from_numpy(rng.standard_normal(n, dtype=np.float32))
    b = T.from_numpy(rng.uniform(0.5, 2.0, n).astype(np.float32))
    y = T.empty((n,))
    for op in ("add", "sub", "mul", "div", "gt"):
        timed(f"{op}_c3_f32", 3.0 * a.nbytes, lambda op=op: lib.call(f"keydnn_cuda_{op}_f32", a.data, b.data, y.data, n))
    timed("neg_c3_f32", 2.0 * a.nbytes, lambda: lib.call("keydnn_cuda_neg_f32", a.data, y.data, n))
    ga, gb = T.empty((n,)), T.empty((n,))
    # backward of mul / div: read g, a, b, write both gradients (5 tensor passes)
    timed("mul_backward_c3_f32", 5.0 * a.nbytes, lambda: lib.call("keydnn_cuda_mul_backward_f32", y.data, a.data, b.data,
                                                                 ga.data, gb.data, n))
    timed("div_backward_c3_f32", 5.0 * a.nbytes, lambda: lib.call("keydnn_cuda_div_backward_f32", y.data, a.data, b.data,
                                                                 ga.data, gb.data, n))
    del a, b, y, ga, gb
    n = 25_165_824
    p = T.from_numpy(rng.standard_normal(n, dtype=np.float32))
    g = T.from_numpy((rng.standard_normal(n, dtype=np.float32) * np.float32(1e-2)))
    v = T.zeros((n,))
    timed("sgd_momentum_step_c3_f32", 5.0 * p.nbytes, lambda: lib.call(
        "keydnn_cuda_sgd_momentum_step_f32", p.data, g.data, v.data, n, ctypes.c_float(0.01), ctypes.c_float(0.9),
        ctypes.c_float(1e-4), ctypes.c_float(1.0)))
    # Adam on the same vector: read p, g, m, v, write p, m, v (7 passes)
    m, v = T.zeros((n,)), T.zeros((n,))          # a fresh second moment: the SGD velocity above has negative entries
    cf = ctypes.c_float
    timed("adam_step_c3_f32", 7.0 * p.nbytes, lambda: lib.call(
        "keydnn_cuda_adam_step_f32", p.data, g.data, m.data, v.data, n, cf(1e-3), cf(0.9), cf(0.999), cf(1e-8), cf(1e-4),
        cf(0.1), cf(0.001), cf(0.1), cf(0.001), cf(1.0)))
    del p, g, v, m
    # activations, softmax and losses on 2^27 fp32 elements (537 MB per tensor)
    n = 1 << 27
    x = T.from_numpy(rng.standard_normal(n, dtype=np.float32))
    y, gx = T.empty((n,)), T.empty((n,))
    xpos = T.from_numpy(np.abs(x.to_numpy()) + np.float32(0.01))      # log / sqrt of positive values (NaN results take a slow path)
    for name in ("exp", "log", "sqrt", "sigmoid_forward", "tanh_forward"):
        count = n if name != "exp" else ctypes.c_int(n)
        src = xpos if name in ("log", "sqrt") else x
        timed(f"{name}_f32", 2.0 * x.nbytes, lambda name=name, count=count, src=src: lib.call(
            f"keydnn_cuda_{name}_f32", src.data, y.data, count))
    del xpos
    timed("relu_forward_f32", 2.0 * x.nbytes, lambda: lib.call("keydnn_cuda_relu_forward_f32", x.data, y.data, None, n))
    timed("leaky_relu_forward_f32", 2.0 * x.nbytes, lambda: lib.call("keydnn_cuda_leaky_relu_forward_f32", x.data, y.data, cf(0.1), n))
    for name in ("sigmoid_backward", "tanh_backward", "relu_backward", "sqrt_backward"):
        timed(f"{name}_f32", 3.0 * x.nbytes, lambda name=name: lib.call(f"keydnn_cuda_{name}_f32", x.data, y.data, gx.data, n))
    for rows_, cols_ in ((1 << 17, 1 << 10), (1 << 23, 16), (1 << 13, 1 << 14)):
        timed(f"softmax_fwd_{rows_}x{cols_}_f32", 2.0 * x.nbytes, lambda r=rows_, c=cols_: lib.call(
            "keydnn_cuda_softmax_forward_f32", x.data, y.data, r, c, 1))
        timed(f"softmax_bwd_{rows_}x{cols_}_f32", 3.0 * x.nbytes, lambda r=rows_, c=cols_: lib.call(
            "keydnn_cuda_softmax_backward_f32", x.data, y.data, gx.data, r, c, 1))
    loss = T.empty(())
    pr = T.from_numpy(rng.uniform(0.05, 0.95, n).astype(np.float32))
    timed("sqdiff_forward_mean_f32", 2.0 * x.nbytes, lambda: lib.call("keydnn_cuda_sqdiff_forward_f32", pr.data, x.data, None,
                                                                     loss.data, n, 1))
    timed("bce_forward_f32", 2.0 * x.nbytes, lambda: lib.call("keydnn_cuda_bce_forward_f32", pr.data, y.data, loss.data, n))
    timed("bce_backward_f32", 3.0 * x.nbytes, lambda: lib.call("keydnn_cuda_bce_backward_f32", pr.data, y.data, None, gx.data, n))
    timed("cce_forward_f32", 2.0 * x.nbytes, lambda: lib.call("keydnn_cuda_cce_forward_f32", pr.data, y.data, loss.data, n, 1 << 17))
    timed("cce_backward_f32", 3.0 * x.nbytes, lambda: lib.call("keydnn_cuda_cce_backward_f32", pr.data, y.data, None, gx.data, n,
                                                             1 << 17))
    del x, y, gx, pr
    # layer glue: bias add, broadcast, un-broadcast, transpose on the CNN's activation shape
    N_, C_, HW_ = 256, 32, 64 * 64
    act = T.from_numpy(rng.standard_normal((N_, C_, HW_), dtype=np.float32))
    out = T.empty(act.shape)
    bias = T.from_numpy(rng.standard_normal(C_, dtype=np.float32))
    i64 = ctypes.c_int64
    in_shape, out_shape = (i64 * 3)(N_, C_, HW_), (i64 * 3)(1, C_, 1)
    chan = T.empty((C_,))
    timed("sum_to_shape_NCHW_to_C_f32", float(act.nbytes), lambda: lib.call(
        "keydnn_cuda_sum_to_shape_f32", act.data, chan.data, in_shape, out_shape, 3))
    timed("broadcast_to_C_to_NCHW_f32", float(act.nbytes), lambda: lib.call(
        "keydnn_cuda_broadcast_to_f32", bias.data, out.data, out_shape, 3, in_shape, 3))
    xb = T.from_numpy(rng.standard_normal((1 << 16, 1024), dtype=np.float32))
    yb = T.empty(xb.shape)
    b1k = T.from_numpy(rng.standard_normal(1024, dtype=np.float32))
    timed("bias_add_65536x1024_f32", 2.0 * xb.nbytes, lambda: lib.call("keydnn_cuda_bias_add_f32", xb.data, b1k.data, yb.data,
                                                                      1 << 16, 1024))
    del xb, yb
    mat = T.from_numpy(rng.standard_normal((8192, 4096), dtype=np.float32))
    matT = T.empty((4096, 8192))
    timed("transpose2d_8192x4096_f32", 2.0 * mat.nbytes, lambda: lib.call("keydnn_cuda_transpose2d_f32", mat.data, matT.data, 8192, 4096))
    return rows


def run_ours(args) -> None:
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import distributed
    from keydnn_v2_b200.sharded import ShardedReductions

    rank, world, local = _env_int("RANK", 0), _env_int("WORLD_SIZE", 1), _env_int("LOCAL_RANK", 0)
    lib = kd.load()
    lib.call("keydnn_cuda_set_device", local)
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
        group = distributed.init_from_torch(device=local)
    else:
        group = distributed.single(lib)

    if args.workload == "cnn":
        timer = Timer(lib)
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        cnn = cnn_step_bench(lib, group, dist, args.steps, args.warmup, timer)
        clocks = sampler.stop() if rank == 0 else None
        if rank == 0:
            print(json.dumps({
                "metric": "CNN training step samples/s (configs[4])", "value": cnn["samples_per_s"], "unit": "samples/s",
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": cnn["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "configs[4]: " + cnn["model"], "global_batch": cnn["batch_per_gpu"] * world,
                           "parallelism": cnn["parallelism"]},
                "e2e": {"value": cnn["e2e_samples_per_s"], "unit": "samples/s",
                        "h2d_bytes_per_step": cnn["h2d_bytes_per_step"], "d2h_bytes_per_step": cnn["d2h_bytes_per_step"]},
                "clocks": clocks, "cnn_step": cnn}), flush=True)
        if dist is not None:
            group.destroy()
            dist.destroy_process_group()
        return

    # everything below runs on a created stream (the legacy default stream cannot be recorded into a graph)
    work_stream = ctypes.c_uint64(0)
    lib.call("keydnn_cuda_stream_create", ctypes.byref(work_stream))
    lib.call("keydnn_cuda_set_stream", work_stream.value)
    rng = np.random.default_rng(1 + rank)
    T = kd.Tensor
    h32 = rng.standard_normal((ROWS32, COLS32), dtype=np.float32)
    h64 = rng.standard_normal((ROWS64, COLS64))
    r32 = ShardedReductions(T.from_numpy(h32), group)
    r64 = ShardedReductions(T.from_numpy(h64), group)
    reducers = [(r32, "f32"), (r64, "f64")]
    timer = Timer(lib)
    launches = [0]

    def step() -> None:
        # all forward reductions, then all backward passes (the order of a graph with eighteen reduction heads);
        # the forward partials cross ranks in one bucket per matrix once the forward kernels are enqueued
        for op, ax in OPS:
            for red, _ in reducers:
                red.forward(op, ax, defer=True)
        for red, _ in reducers:
            red.flush()                  # one all-reduce + one all-gather per matrix, under the backward kernels
        for op, ax in OPS:
            for red, _ in reducers:
                red.backward(op, ax)
        for red, _ in reducers:
            red.finish()                 # the step ends when its collectives have landed
        launches[0] += 2 * len(OPS) * len(reducers)

    def barrier() -> None:
        lib.call("keydnn_cuda_synchronize")
        if dist is not None:
            dist.barrier()

    if args.once:
        # one launch of every kernel, for a profiler capture (`ncu -k ... python bench.py --once`)
        step()
        lib.call("keydnn_cuda_synchronize")
        del r32, r64, reducers
        lib.call("keydnn_cuda_empty_cache")
        suite_table(lib, timer, 1.0, reps=1, warm=0)
        lib.call("keydnn_cuda_synchronize")
        print("once: every kernel launched one time", flush=True)
        return

    # the clock sampler (one nvidia-smi process) is started before the warm-up: its start-up talks to the driver
    # for tens of ms and must not fall into the K timed steps; its samples are kept from the end of the warm-up on
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # At N > 1 the step (kernels, the second stream's collectives, the events between them) is recorded once and
    # replayed with one launch per step: the ranks meet in four collectives per step, so a rank whose host thread
    # is late with its ~120 enqueue calls holds all of them up; a replay takes the host out of the loop.
    # (At N = 1 nothing waits on another process and the eager enqueue is far ahead of the GPU.)
    run_step, stepping, step_graph = step, "eager", ctypes.c_uint64(0)
    if world > 1:
        try:
            lib.call("keydnn_cuda_graph_capture_begin")
            try:
                step()
            finally:
                lib.call("keydnn_cuda_graph_capture_end", ctypes.byref(step_graph))
            per_step = 2 * len(OPS) * len(reducers)

            def run_step() -> None:
                lib.call("keydnn_cuda_graph_launch", step_graph.value)
                launches[0] += per_step

            stepping = "cuda graph replay"
            for _ in range(2):
                run_step()
        except Exception as exc:  # noqa: BLE001
            run_step, stepping = step, f"eager (graph capture failed: {type(exc).__name__})"
        flags = [stepping]
        if dist is not None:
            gathered = [None] * world
            dist.all_gather_object(gathered, stepping)
            flags = gathered
        if any(f != "cuda graph replay" for f in flags):        # all ranks replay, or none does
            run_step, stepping = step, "eager"
        barrier()
    sampler.mark()
    launches[0] = 0
    # the host only enqueues; a cyclic-collector pass of the interpreter (tens of ms once torch is imported at N > 1)
    # inside K steps of ~1 ms would starve the GPU, so the collector is paused for the timed regions
    gc.collect()
    gc.disable()
    timer.start()
    for _ in range(args.steps):
        run_step()
    ms = timer.stop_ms()
    barrier()
    n_launch = launches[0]
    if step_graph.value:
        lib.call("keydnn_cuda_graph_destroy", step_graph.value)

    # ---- end to end: pinned host inputs in, results out, through the public Tensor API ----
    def pinned_like(a: np.ndarray) -> np.ndarray:
        p = ctypes.c_void_p(0)
        lib.call("keydnn_cuda_host_alloc", ctypes.byref(p), a.nbytes)
        buf = (ctypes.c_char * a.nbytes).from_address(p.value)
        out = np.frombuffer(buf, dtype=a.dtype).reshape(a.shape)
        out[...] = a
        return out

    p32, p64 = pinned_like(h32), pinned_like(h64)
    del h32, h64
    host_out = {id(r32): np.empty(max(ROWS32, COLS32), np.float32), id(r64): np.empty(max(ROWS64, COLS64), np.float64)}
    d2h = [0]

    # host -> device copies go on their own stream: the second matrix is still arriving while the
    # kernels of the first one run; results are read back once all kernels of the step are enqueued
    main_stream, copy_stream = ctypes.c_uint64(0), ctypes.c_uint64(0)
    lib.call("keydnn_cuda_get_stream", ctypes.byref(main_stream))
    lib.call("keydnn_cuda_stream_create", ctypes.byref(copy_stream))
    arrived = []
    for _ in reducers:
        e = ctypes.c_uint64(0)
        lib.call("keydnn_cuda_event_create", ctypes.byref(e))
        arrived.append(e.value)

    def e2e_step() -> None:
        d2h[0] = 0
        lib.call("keydnn_cuda_set_stream", copy_stream.value)
        for (red, _), src, ev in zip(reducers, (p32, p64), arrived):
            lib.call("keydnn_cuda_memcpy_h2d_async", red.x.data, src.ctypes.data, src.nbytes)
            lib.call("keydnn_cuda_event_record", ev)
        lib.call("keydnn_cuda_set_stream", main_stream.value)
        results = []
        for (red, _), ev in zip(reducers, arrived):
            lib.call("keydnn_cuda_stream_wait_event", ev)
            for op, ax in OPS:
                ptr, n = red.forward(op, ax)
                red.backward(op, ax)
                results.append((red, op, ax, ptr, n))
        for red, op, ax, ptr, n in results:
            red.wait(op, ax)
            nb = n * red.dt.itemsize
            lib.call("keydnn_cuda_memcpy_d2h", host_out[id(red)].ctypes.data, ptr, nb)
            d2h[0] += nb
        for red, _ in reducers:      # the step's gradient result: first row of the last gradient
            lib.call("keydnn_cuda_memcpy_d2h", host_out[id(red)].ctypes.data, red.gx.data, red.cols * red.dt.itemsize)
            d2h[0] += red.cols * red.dt.itemsize

    e2e_step()
    barrier()
    gc.collect()
    e2e_steps = max(2, min(args.steps, 5))
    t0 = time.perf_counter()
    timer.start()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_ms = timer.stop_ms()
    e2e_wall = (time.perf_counter() - t0) * 1e3
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    if dist is not None:
        import torch

        t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    # per-kernel timings run on every rank; rank 0 reports its own
    peak, peak_src = measured_peak_gbs()
    # (at N > 1 the table times the local kernels alone: same shards, no exchange behind them)
    local = reducers if world == 1 else [(ShardedReductions(red.x, distributed.single(lib)), tag) for red, tag in reducers]
    table = kernel_table(lib, local, timer, 20, peak) if args.kernels != "none" else None
    del local
    suite = suite_table(lib, timer, peak) if args.kernels == "suite" else None
    line = None
    if rank == 0:
        bytes_step = algorithmic_bytes_per_step()
        value = bytes_step * world * args.steps / ms / 1e6
        e2e_val = bytes_step * world * e2e_steps / max(e2e_ms, e2e_wall) / 1e6
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32+f64", "data": "synthetic",
            "config": {"workload": "configs[1]: sum/mean/max over axis 0, axis 1, all axes, fwd + bwd (grad of ones), "
                                   "fp32 (8192,8192) N(0,1) + fp64 (4096,4096) N(0,1) per GPU, rows sharded across GPUs",
                       "l2": "inputs larger than L2 (268 MB and 134 MB vs 126 MB); no flush",
                       "collectives": "none" if world == 1 else "NCCL all-reduce / all-gather of axis-0 and all-axes partials, "
                                                                 "one bucket of each per matrix and step",
                       "stepping": stepping},
            "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": int(p32.nbytes + p64.nbytes),
                    "d2h_bytes_per_step": int(d2h[0]), "steps": e2e_steps},
            "gpu_launches": n_launch, "clocks": clocks,
        }
        if table is not None:
            top = max(table, key=lambda r: r["us"])
            line["roofline"] = {"bound": "hbm", "kernel": top["kernel"], "achieved": top["gbs"], "peak": peak,
                                "unit": "GB/s", "frac": top["frac"], "traffic": NCU_TRAFFIC_BYTES.get(top["kernel"]),
                                "traffic_unit": "bytes per launch (ncu dram read+write, captured once; summary under profiles/)",
                                "algorithmic_bytes": top["bytes"], "peak_source": peak_src,
                                "frac_of_nominal_8000": round(top["gbs"] / 8000.0, 4)}
            line["kernels"] = table
            if suite is not None:
                line["suite"] = suite
            line["whole_step_frac"] = round(value / world / peak, 4)
        # timed at N = 1 only: at N > 1 the other ranks would sit in the next collective while rank 0 computes
        line["cpu_baseline"] = cpu_baseline_sample() if world == 1 else None
    cnn = None
    if args.cnn != "off":
        del r32, r64, reducers
        lib.call("keydnn_cuda_empty_cache")
        cnn = cnn_step_bench(lib, group, dist, max(args.steps, 10), args.warmup, timer)
    if rank == 0:
        line["cnn_step"] = cnn
        print(json.dumps(line), flush=True)
    if dist is not None:
        group.destroy()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# configs[4]: small-CNN training step, data parallel
# ---------------------------------------------------------------------------
def cnn_step_bench(lib, group, dist, steps: int, warmup: int, timer, batch: int = 256) -> dict:
    """Conv-BN-ReLU-MaxPool-Conv-BN-ReLU-GlobalAvgPool-Flatten-Linear, MSE, SGD-momentum; batch 256 per GPU,
    per-shard BatchNorm, one gradient all-reduce per step.  Returns samples/s with inputs resident and
    end to end (pinned host batch copied in, loss copied out, every step)."""
    import keydnn_v2_b200 as kd
    from keydnn_v2_b200 import nn

    rank, world = group.rank, group.world
    np.random.seed(1234)                         # same initial weights on every rank
    model = nn.small_cnn()
    opt = nn.SGD(model.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4, group=group)
    rng = np.random.default_rng(100 + rank)
    def pinned(a: np.ndarray) -> np.ndarray:
        p = ctypes.c_void_p(0)
        lib.call("keydnn_cuda_host_alloc", ctypes.byref(p), a.nbytes)
        out = np.frombuffer((ctypes.c_char * a.nbytes).from_address(p.value), dtype=a.dtype).reshape(a.shape)
        out[...] = a
        return out

    hx = pinned(rng.standard_normal((batch, 3, 64, 64), dtype=np.float32))
    ht = pinned(np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)])
    x, t = kd.Tensor.from_numpy(hx), kd.Tensor.from_numpy(ht)

    def sync() -> None:
        lib.call("keydnn_cuda_synchronize")
        if dist is not None:
            dist.barrier()

    for _ in range(max(warmup, 3)):
        loss = nn.train_step(model, opt, x, t)
    first = loss.item()
    sync()
    # the step is recorded into a CUDA graph (one launch per step); eager stepping is the fallback
    graph, graph_note = None, "cuda graph replay"
    try:
        graph = nn.GraphedTrainStep(model, opt, x, t, warmup=2)
        run_step = graph.run
    except Exception as exc:  # noqa: BLE001
        graph_note = f"eager (graph capture failed: {type(exc).__name__})"

        def run_step():
            return nn.train_step(model, opt, x, t)

    for _ in range(3):
        loss = run_step()
    sync()
    gc.collect()
    gc.disable()            # see run_ours: no collector pass inside the timed steps
    timer.start()
    for _ in range(steps):
        loss = run_step()
    ms = timer.stop_ms()
    sync()
    last = loss.item()
    if graph is not None:
        graph.loss_of(graph.step_async(hx, ht))     # builds the copy stream, events and staging buffers: not timed
        sync()
    t0 = time.perf_counter()
    timer.start()
    if graph is not None:
        # the public pipelined call: batch i+1 crosses PCIe on a copy stream while step i replays; every step's
        # loss is copied to the host and read there one step later
        pending = None
        for _ in range(steps):
            ticket = graph.step_async(hx, ht)
            if pending is not None:
                graph.loss_of(pending)
            pending = ticket
        graph.loss_of(pending)
    else:
        for _ in range(steps):
            lib.call("keydnn_cuda_memcpy_h2d_async", x.data, hx.ctypes.data, hx.nbytes)
            lib.call("keydnn_cuda_memcpy_h2d_async", t.data, ht.ctypes.data, ht.nbytes)
            loss = run_step()
            loss.item()
    e2e_ms = max(timer.stop_ms(), (time.perf_counter() - t0) * 1e3)
    sync()
    if graph is not None:
        graph.close()
    if dist is not None:
        import torch

        tt = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(tt[0]), float(tt[1])
    return {"samples_per_s": round(batch * world * steps / ms * 1e3, 1), "ms_per_step": round(ms / steps, 4),
            "e2e_samples_per_s": round(batch * world * steps / e2e_ms * 1e3, 1), "batch_per_gpu": batch, "steps": steps,
            "h2d_bytes_per_step": int(hx.nbytes + ht.nbytes), "d2h_bytes_per_step": 4,
            "loss_first": round(first, 6), "loss_last": round(last, 6), "stepping": graph_note,
            "model": "Conv(3-32)-BN-ReLU-MaxPool2-Conv(32-64)-BN-ReLU-GAP-Flatten-Linear(64-10), MSE, SGD momentum 0.9 wd 1e-4",
            "parallelism": f"dp{world}, per-shard BatchNorm, one NCCL all-reduce of the flat gradient buffer per step"}


# ---------------------------------------------------------------------------
# CPU baseline and the reference arm
# ---------------------------------------------------------------------------
def cpu_baseline_sample(rows32: int = ROWS32 // 4, rows64: int = ROWS64 // 4, budget_s: float = 12.0) -> dict:
    """The reference's CPU path (single-threaded NumPy expressions) on a quarter of the rows of the configs[1]
    matrices, repeated until about `budget_s` seconds of CPU work have been timed."""
    from oracle import cpu_baseline

    rng = np.random.default_rng(1)
    x32 = rng.standard_normal((rows32, COLS32), dtype=np.float32)
    x64 = rng.standard_normal((rows64, COLS64))
    cpu_baseline.time_reduce_workload(x32[:64], x64[:64])
    nbytes = seconds = 0.0
    passes = 0
    while seconds < budget_s and passes < 48:
        r = cpu_baseline.time_reduce_workload(x32, x64)
        nbytes += r["bytes"]
        seconds += r["seconds"]
        passes += 1
    return {"value": round(nbytes / seconds / 1e9, 3), "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"{passes} passes over a quarter of the rows ({rows32}x{COLS32} fp32 + {rows64}x{COLS64} fp64, all 9 reductions "
                      f"fwd+bwd), {seconds:.1f} s; NumPy expressions of the reference's CPU Tensor methods",
            "host_cores": os.cpu_count()}


def run_reference(args) -> None:
    rank, world = _env_int("RANK", 0), _env_int("WORLD_SIZE", 1)
    if rank != 0:
        return
    from oracle import cpu_baseline

    rng = np.random.default_rng(1)
    rows32, rows64 = ROWS32 // 4, ROWS64 // 4          # one step = a quarter of the rows, about a second of CPU work
    x32 = rng.standard_normal((rows32, COLS32), dtype=np.float32)
    x64 = rng.standard_normal((rows64, COLS64))
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_baseline.time_reduce_workload(x32, x64)
    t0 = time.perf_counter()
    nbytes = 0.0
    for _ in range(args.steps):
        nbytes += cpu_baseline.time_reduce_workload(x32, x64)["bytes"]
    dt = time.perf_counter() - t0
    value = nbytes / dt / 1e9
    sample = (f"each step = a quarter of the rows ({rows32}x{COLS32} fp32 + {rows64}x{COLS64} fp64, all 9 reductions fwd+bwd) "
              "on the host cores (NumPy is single-threaded for these expressions)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+f64", "data": "synthetic",
        "config": {"workload": "configs[1] reductions fwd+bwd, CPU path of the reference (NumPy)"},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample,
                         "host_cores": os.cpu_count()},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernels", default="all", choices=["all", "none", "suite"])
    ap.add_argument("--workload", default="reduce", choices=["reduce", "cnn"],
                    help="reduce: configs[1] (the default line); cnn: only the configs[4] training step, reported as samples/s")
    ap.add_argument("--cnn", default="on", choices=["on", "off"], help="also time the small-CNN training step (configs[4])")
    ap.add_argument("--once", action="store_true", help="launch every kernel once and exit (profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
