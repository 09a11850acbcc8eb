"""The allocation-free column-sum entry point (keydnn_cuda_sum_axis0_noalloc_f32).

Some callers cannot let a library allocate device memory when they call it: a host framework
whose caching allocator already owns the device heap, a serving loop that must not stall on the
allocator, a process with a fixed memory budget.  For them this entry keeps its partial sums in
a static device array instead of the library's growable scratch buffer.  It must give what the
regular entry (keydnn_cuda_sum_axis2d_forward_f32, axis 0) gives, call after call: the static
array keeps the previous call's contents, so the second call of each pair below runs on a dirty
array, with another shape.  Collected last so that a failure here cannot hide other failures.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from _gpu_util import Buf, native

pytestmark = pytest.mark.gpu

TOL = dict(rtol=1e-5, atol=1e-5)


def _both(lib, x):
    rows, cols = x.shape
    dx = Buf(lib, x)
    y_ref, y_new = Buf(lib, shape=(cols,), dtype=np.float32, fill=0xFF), Buf(lib, shape=(cols,), dtype=np.float32, fill=0xFF)
    lib.call("keydnn_cuda_sum_axis2d_forward_f32", dx.ptr, y_ref.ptr, rows, cols, 0)
    lib.call("keydnn_cuda_sum_axis0_noalloc_f32", dx.ptr, y_new.ptr, rows, cols)
    return y_ref.get(), y_new.get()


@pytest.mark.parametrize("shapes", [((2048, 4096), (777, 1000)), ((5, 3), (4096, 8192)), ((3000, 264), (3000, 260))])
def test_two_calls_in_a_row_match_the_regular_entry(shapes):
    lib = native()
    rng = np.random.default_rng(12)
    for shape in shapes:
        x = rng.standard_normal(shape).astype(np.float32)
        ref, new = _both(lib, x)
        np.testing.assert_allclose(new, ref, **TOL)
        np.testing.assert_allclose(new, x.astype(np.float64).sum(axis=0), rtol=1e-5, atol=1e-4)


_FIRST_CALL = r"""
import ctypes, sys
import numpy as np
sys.path.insert(0, sys.argv[1])
import keydnn_v2_b200 as kd
lib = kd.load()
def scratch_allocs():
    out = (ctypes.c_uint64 * 4)()
    lib.call("keydnn_cuda_scratch_stats", out)
    return int(out[2])
x = np.ones((1024, 2048), np.float32)
px, py = ctypes.c_uint64(0), ctypes.c_uint64(0)
lib.call("keydnn_cuda_malloc", ctypes.byref(px), x.nbytes)
lib.call("keydnn_cuda_malloc", ctypes.byref(py), 2048 * 4)
lib.call("keydnn_cuda_memcpy_h2d", px.value, x.ctypes.data, x.nbytes)
for _ in range(2):
    lib.call("keydnn_cuda_sum_axis0_noalloc_f32", px.value, py.value, 1024, 2048)
a = scratch_allocs()
lib.call("keydnn_cuda_sum_axis2d_forward_f32", px.value, py.value, 1024, 2048, 0)
print("allocs", a, scratch_allocs())
"""


def _mem_state(lib):
    pool, scratch, mem = (ctypes.c_uint64 * 4)(), (ctypes.c_uint64 * 4)(), (ctypes.c_uint64 * 2)()
    lib.call("keydnn_cuda_pool_stats", pool)
    lib.call("keydnn_cuda_scratch_stats", scratch)
    lib.call("keydnn_cuda_mem_info", mem)
    return list(pool), list(scratch), int(mem[0])


def test_makes_no_device_allocation():
    """Three things may not move across calls of the entry: the caching pool's driver allocations, the
    allocations made for the growable reduction scratch (the regular entry's partials live there, and its
    `cudaMalloc` goes around the pool), and the free device memory the driver reports."""
    lib = native()
    x = np.ones((1024, 2048), np.float32)
    dx, dy = Buf(lib, x), Buf(lib, shape=(2048,), dtype=np.float32)
    lib.call("keydnn_cuda_sum_axis0_noalloc_f32", dx.ptr, dy.ptr, 1024, 2048)     # first call: address look-up
    lib.call("keydnn_cuda_synchronize")
    before = _mem_state(lib)
    for _ in range(3):
        lib.call("keydnn_cuda_sum_axis0_noalloc_f32", dx.ptr, dy.ptr, 1024, 2048)
    lib.call("keydnn_cuda_synchronize")
    after = _mem_state(lib)
    assert after[:2] == before[:2]
    assert after[2] >= before[2]              # free device memory did not shrink
    np.testing.assert_array_equal(dy.get(), np.full(2048, 1024.0, np.float32))


def test_the_measure_moves_for_the_regular_entry_in_a_fresh_process():
    """The scratch-allocation count used above is not blind: in a process that has run no reduction yet the
    allocation-free entry leaves it at zero and the first call of the regular entry raises it."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    repo = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, "-c", _FIRST_CALL, str(repo)], capture_output=True, text=True,
                       env=dict(os.environ), timeout=300)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-3000:]
    tag, a, b = r.stdout.split()[-3:]
    assert tag == "allocs" and int(a) == 0 and int(b) >= 1, r.stdout


def test_rejects_sizes_beyond_the_static_array():
    lib = native()
    d = Buf(lib, np.zeros(16, np.float32))
    f = lib.raw("keydnn_cuda_sum_axis0_noalloc_f32")
    assert f(d.ptr, d.ptr, 4, 65537) == -20          # launches nothing
    assert f(None, d.ptr, 4, 4) == -1
    assert f(d.ptr, d.ptr, 0, 4) == -2
