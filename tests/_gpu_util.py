"""Helpers for the GPU parity tests: device buffers through the C ABI, and the two
checkers (the CPU oracle and the reference's own CUDA kernels compiled unmodified)."""
from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[1]
REF_CUDA = REPO / "oracle" / "_ref" / "libkeydnn_ref_cuda.so"


@lru_cache(maxsize=1)
def native():
    from keydnn_v2_b200 import load

    return load()


@lru_cache(maxsize=1)
def ref_cuda():
    """The reference's CUDA library (same C ABI), or None when it was not built."""
    if not REF_CUDA.exists():
        return None
    from keydnn_v2_b200._native import Native

    return Native(REF_CUDA, strict=False)


GUARD = 256                 # bytes of sentinel on each side of every test buffer
SENTINEL = 0xA5
OVERRUNS: list[str] = []    # guard bands found damaged (tests/conftest.py fails the test that left an entry)


class Buf:
    """A device buffer owned by `lib` (either library: both export malloc/free/memcpy).

    The allocation carries a guard band of `GUARD` sentinel bytes directly in front of the buffer and directly
    behind its last byte.  The caching pool rounds sizes up (512-byte classes), so a kernel that writes a few
    elements past the end of a ragged buffer would otherwise land in slack that nobody reads; the bands are
    compared on every `get()` and when the buffer is released, which stands in for a memory checker."""

    def __init__(self, lib, arr=None, *, shape=None, dtype=None, fill=None):
        self.lib = lib
        if arr is not None:
            arr = np.ascontiguousarray(arr)
            shape, dtype = arr.shape, arr.dtype
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        out = ctypes.c_uint64(0)
        lib.call("keydnn_cuda_malloc", ctypes.byref(out), GUARD + max(self.nbytes, 16) + GUARD)
        self.base = out.value
        self.ptr = self.base + GUARD          # still 256-byte aligned
        lib.call("keydnn_cuda_memset", self.base, SENTINEL, GUARD)
        lib.call("keydnn_cuda_memset", self.ptr + self.nbytes, SENTINEL, GUARD)
        if arr is not None and self.nbytes:
            lib.call("keydnn_cuda_memcpy_h2d", self.ptr, arr.ctypes.data, self.nbytes)
        elif fill is not None and self.nbytes:
            lib.call("keydnn_cuda_memset", self.ptr, int(fill), self.nbytes)

    def check_guards(self) -> None:
        """Records (and raises on) any byte of either guard band that no longer holds the sentinel."""
        band = np.empty(GUARD, np.uint8)
        self.lib.call("keydnn_cuda_synchronize")
        for name, addr in (("in front of", self.base), ("behind", self.ptr + self.nbytes)):
            self.lib.call("keydnn_cuda_memcpy_d2h", band.ctypes.data, addr, GUARD)
            bad = np.flatnonzero(band != SENTINEL)
            if bad.size:
                msg = (f"out-of-bounds write {name} a {self.shape} {self.dtype} buffer: {bad.size} guard bytes changed, "
                       f"first at offset {int(bad[0])}")
                OVERRUNS.append(msg)
                raise AssertionError(msg)

    def get(self) -> np.ndarray:
        out = np.empty(self.shape, self.dtype)
        self.check_guards()
        if self.nbytes:
            self.lib.call("keydnn_cuda_memcpy_d2h", out.ctypes.data, self.ptr, self.nbytes)
        return out

    def __del__(self):
        try:
            self.check_guards()
        except Exception:
            pass                               # recorded in OVERRUNS; the fixture fails the test
        try:
            self.lib.raw("keydnn_cuda_free")(ctypes.c_uint64(self.base))
        except Exception:
            pass


def suf(dtype) -> str:
    return "f32" if np.dtype(dtype) == np.float32 else "f64"


def cfloat(dtype, v):
    return ctypes.c_float(v) if np.dtype(dtype) == np.float32 else ctypes.c_double(v)


def bits(a: np.ndarray) -> np.ndarray:
    """Integer view for bit-exact comparison (distinguishes -0.0 and NaN payloads)."""
    a = np.ascontiguousarray(a)
    return a.view(np.uint32 if a.dtype == np.float32 else np.uint64)


TOL = {np.dtype(np.float32): dict(rtol=1e-5, atol=1e-6), np.dtype(np.float64): dict(rtol=1e-12, atol=1e-12)}


def assert_same_bits(got: np.ndarray, want: np.ndarray, err_msg: str = "") -> None:
    """Bit-exact equality (so -0.0 != +0.0), except that any NaN matches any NaN: CPUs
    propagate an input NaN's payload, GPUs return the canonical NaN."""
    assert got.dtype == want.dtype and got.shape == want.shape, (got.dtype, want.dtype, got.shape, want.shape)
    gn, wn = np.isnan(got), np.isnan(want)
    np.testing.assert_array_equal(gn, wn, err_msg=err_msg + " (NaN positions)")
    np.testing.assert_array_equal(bits(np.where(gn, 0, got).astype(got.dtype)),
                                  bits(np.where(wn, 0, want).astype(want.dtype)), err_msg=err_msg)
