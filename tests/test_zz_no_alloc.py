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


def test_makes_no_device_allocation():
    lib = native()
    x = np.ones((1024, 2048), np.float32)
    dx, dy = Buf(lib, x), Buf(lib, shape=(2048,), dtype=np.float32)
    lib.call("keydnn_cuda_sum_axis0_noalloc_f32", dx.ptr, dy.ptr, 1024, 2048)     # first call: address look-up
    before = (ctypes.c_uint64 * 4)()
    after = (ctypes.c_uint64 * 4)()
    lib.call("keydnn_cuda_pool_stats", before)
    for _ in range(3):
        lib.call("keydnn_cuda_sum_axis0_noalloc_f32", dx.ptr, dy.ptr, 1024, 2048)
    lib.call("keydnn_cuda_pool_stats", after)
    assert list(before) == list(after)
    np.testing.assert_array_equal(dy.get(), np.full(2048, 1024.0, np.float32))


def test_rejects_sizes_beyond_the_static_array():
    lib = native()
    d = Buf(lib, np.zeros(16, np.float32))
    f = lib.raw("keydnn_cuda_sum_axis0_noalloc_f32")
    assert f(d.ptr, d.ptr, 4, 65537) == -20          # launches nothing
    assert f(None, d.ptr, 4, 4) == -1
    assert f(d.ptr, d.ptr, 0, 4) == -2
