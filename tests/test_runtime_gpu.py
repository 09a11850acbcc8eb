"""Runtime behaviour behind the C ABI that only shows with a device: reduction scratch and recorded graphs,
cached blocks that change stream."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from _gpu_util import Buf, native

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parents[1]

_SCRATCH_AND_GRAPH = r"""
import ctypes, sys
import numpy as np
sys.path.insert(0, sys.argv[1])
import keydnn_v2_b200 as kd
lib = kd.load()
u64 = ctypes.c_uint64
def stats():
    out = (u64 * 4)()
    lib.call("keydnn_cuda_scratch_stats", out)
    return list(out)
def dev(a):
    p = u64(0)
    lib.call("keydnn_cuda_malloc", ctypes.byref(p), a.nbytes)
    lib.call("keydnn_cuda_memcpy_h2d", p.value, a.ctypes.data, a.nbytes)
    return p.value
def host(p, n):
    out = np.empty(n, np.float32)
    lib.call("keydnn_cuda_memcpy_d2h", out.ctypes.data, p, out.nbytes)
    return out
stream = u64(0)
lib.call("keydnn_cuda_stream_create", ctypes.byref(stream))
lib.call("keydnn_cuda_set_stream", stream.value)
rng = np.random.default_rng(0)
small = rng.standard_normal((64, 256)).astype(np.float32)
big = rng.standard_normal((4096, 1024)).astype(np.float32)
dx, dy = dev(small), dev(np.zeros(256, np.float32))
bx, by = dev(big), dev(np.zeros(1024, np.float32))
assert stats()[2] == 0
lib.call("keydnn_cuda_sum_axis2d_forward_f32", dx, dy, 64, 256, 0)          # eager first: scratch and tickets appear
s0 = stats()
assert s0[0] == 4096 and s0[2] == 2 and s0[3] == 0, s0
lib.call("keydnn_cuda_graph_capture_begin")
lib.call("keydnn_cuda_sum_axis2d_forward_f32", dx, dy, 64, 256, 0)
# a shape that needs more scratch than there is cannot be recorded: it fails instead of allocating in the recording
st = lib.raw("keydnn_cuda_sum_axis2d_forward_f32")(bx, by, 4096, 1024, 0)
assert st == 2, st                                                           # cudaErrorMemoryAllocation
exe = u64(0)
lib.call("keydnn_cuda_graph_capture_end", ctypes.byref(exe))
assert stats() == s0
# a larger eager reduction outgrows the buffer while the graph is alive: the old one is parked, not freed
lib.call("keydnn_cuda_sum_axis2d_forward_f32", bx, by, 4096, 1024, 0)
s1 = stats()
assert s1[0] >= 128 * 1024 * 4 and s1[2] == 3 and s1[3] == 1, s1
np.testing.assert_allclose(host(by, 1024), big.astype(np.float64).sum(0), rtol=1e-5, atol=1e-4)
# the replay still writes its partials to the address it recorded
fresh = rng.standard_normal((64, 256)).astype(np.float32)
lib.call("keydnn_cuda_memcpy_h2d", dx, fresh.ctypes.data, fresh.nbytes)
for _ in range(3):
    lib.call("keydnn_cuda_graph_launch", exe.value)
    lib.call("keydnn_cuda_sum_axis2d_forward_f32", bx, by, 4096, 1024, 0)  # eager work in between, on the new buffer
np.testing.assert_allclose(host(dy, 256), fresh.astype(np.float64).sum(0), rtol=1e-5, atol=1e-5)
np.testing.assert_allclose(host(by, 1024), big.astype(np.float64).sum(0), rtol=1e-5, atol=1e-4)
lib.call("keydnn_cuda_graph_destroy", exe.value)
assert stats()[3] == 0
lib.call("keydnn_cuda_sum_axis2d_forward_f32", dx, dy, 64, 256, 0)
np.testing.assert_allclose(host(dy, 256), fresh.astype(np.float64).sum(0), rtol=1e-5, atol=1e-5)
print("scratch-and-graph ok")
"""


def _child(script: str, **env) -> str:
    e = dict(os.environ, **env)
    r = subprocess.run([sys.executable, "-c", script, str(REPO)], capture_output=True, text=True, env=e, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout


def test_scratch_outgrown_while_a_graph_is_alive_is_parked_and_growth_is_refused_while_recording():
    """A recorded reduction keeps the scratch address it was recorded with.  Run in a fresh process with a
    4 KiB first scratch size so that a second, larger reduction has to grow the buffer: during the recording
    the growth is refused (status 2, nothing allocated inside the recording); after it the old buffer is
    parked until the graph is destroyed and replays keep giving the right sums."""
    assert "scratch-and-graph ok" in _child(_SCRATCH_AND_GRAPH, KEYDNN_B200_SCRATCH_MIN="4096")


def test_cached_block_handed_to_another_stream_waits_for_the_old_one():
    """A block freed under stream A and handed out again under stream B: the kernel on B must not start before
    the work on A that still reads the block.  A long kernel chain on A reads a buffer; the buffer is freed and
    its block reused on B for a fill; the result computed on A must be the one of the original contents."""
    import ctypes

    lib = native()
    n = 1 << 24
    a, b = ctypes.c_uint64(0), ctypes.c_uint64(0)
    prev = ctypes.c_uint64(0)
    lib.call("keydnn_cuda_get_stream", ctypes.byref(prev))
    lib.call("keydnn_cuda_stream_create", ctypes.byref(a))
    lib.call("keydnn_cuda_stream_create", ctypes.byref(b))
    try:
        lib.call("keydnn_cuda_synchronize")
        lib.call("keydnn_cuda_set_stream", a.value)
        ones = np.ones(n, np.float32)
        src, again = ctypes.c_uint64(0), ctypes.c_uint64(0)
        lib.call("keydnn_cuda_malloc", ctypes.byref(src), ones.nbytes)          # raw calls: no host wait anywhere below
        lib.call("keydnn_cuda_memcpy_h2d", src.value, ones.ctypes.data, ones.nbytes)
        acc = Buf(lib, np.zeros(n, np.float32))
        for _ in range(200):                       # about a millisecond of work on A that reads src
            lib.call("keydnn_cuda_add_inplace_f32", acc.ptr, src.value, n)
        lib.call("keydnn_cuda_free", src.value)    # back to the pool, tagged with stream A; the adds are still running
        lib.call("keydnn_cuda_set_stream", b.value)
        lib.call("keydnn_cuda_malloc", ctypes.byref(again), ones.nbytes)        # same size class: the same block
        assert again.value == src.value
        lib.call("keydnn_cuda_memset", again.value, 0, ones.nbytes)             # on B: must wait for the adds on A
        lib.call("keydnn_cuda_synchronize")
        lib.call("keydnn_cuda_set_stream", a.value)
        np.testing.assert_array_equal(acc.get(), np.full(n, 200.0, np.float32))
        lib.call("keydnn_cuda_free", again.value)
    finally:
        lib.call("keydnn_cuda_synchronize")
        lib.call("keydnn_cuda_set_stream", prev.value)
        lib.call("keydnn_cuda_stream_destroy", a.value)
        lib.call("keydnn_cuda_stream_destroy", b.value)


def test_copies_are_bounded_by_the_requested_size_not_the_pool_block():
    """A 40-byte allocation sits in a 512-byte pool block.  cudaMemcpy on a plain cudaMalloc'ed buffer rejects a
    range that leaves the allocation, and the reference's wrappers use that as a size probe
    (ops/matmul_cuda.py reads the last byte each operand should have); the pool must give the same answer."""
    import ctypes

    lib = native()
    p = ctypes.c_uint64(0)
    lib.call("keydnn_cuda_malloc", ctypes.byref(p), 40)
    host = np.zeros(64, np.uint8)
    try:
        d2h, h2d = lib.raw("keydnn_cuda_memcpy_d2h"), lib.raw("keydnn_cuda_memcpy_h2d")
        assert d2h(host.ctypes.data, p.value, 40) == 0
        assert d2h(host.ctypes.data, p.value + 39, 1) == 0
        assert d2h(host.ctypes.data, p.value + 59, 1) == 1            # cudaErrorInvalidValue, as from the driver
        assert d2h(host.ctypes.data, p.value, 41) == 1
        assert h2d(p.value + 8, host.ctypes.data, 33) == 1
        assert lib.raw("keydnn_cuda_memset")(p.value, 0, 64) == 1
        assert lib.raw("keydnn_cuda_memcpy_d2d")(p.value, p.value + 20, 21) == 2
        assert lib.raw("keydnn_cuda_memcpy_d2d")(p.value, p.value + 20, 20) == 0
    finally:
        lib.call("keydnn_cuda_free", p.value)
