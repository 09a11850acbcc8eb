"""Owner of one device allocation.

Mirror of the reference's ``_CudaStorage``
(``src/keydnn/infrastructure/tensor/_cuda_storage.py:86-239``): explicit
``incref``/``decref`` plus a ``weakref.finalize`` safety net, freeing through
``keydnn_cuda_free``.  Here the free returns the block to the library's caching
pool instead of calling ``cudaFree``, so dropping a temporary costs no device
synchronisation.
"""
from __future__ import annotations

import ctypes
import weakref

import numpy as np

from ._native import Native, load


def _release(native: Native, ptr: int) -> None:
    try:
        native.raw("keydnn_cuda_free")(ctypes.c_uint64(ptr))
    except Exception:  # interpreter shutdown
        pass


class CudaStorage:
    __slots__ = ("native", "device_index", "dev_ptr", "nbytes", "dtype", "_refcnt", "_finalizer", "__weakref__")

    def __init__(self, native: Native, device_index: int, dev_ptr: int, nbytes: int, dtype) -> None:
        self.native = native
        self.device_index = int(device_index)
        self.dev_ptr = int(dev_ptr)
        self.nbytes = int(nbytes)
        self.dtype = np.dtype(dtype)
        self._refcnt = 1
        self._finalizer = weakref.finalize(self, _release, native, self.dev_ptr) if self.dev_ptr else None

    @classmethod
    def allocate(cls, nbytes: int, dtype, device_index: int = 0, native: Native | None = None) -> "CudaStorage":
        native = native or load()
        out = ctypes.c_uint64(0)
        native.call("keydnn_cuda_malloc", ctypes.byref(out), ctypes.c_size_t(max(int(nbytes), 1)))
        if out.value == 0:
            raise RuntimeError("keydnn_cuda_malloc returned a null pointer")
        return cls(native, device_index, out.value, nbytes, dtype)

    def incref(self) -> None:
        self._refcnt += 1

    def decref(self) -> None:
        self._refcnt -= 1
        if self._refcnt <= 0:
            self.free()

    def free(self) -> None:
        if self._finalizer is not None and self._finalizer.alive:
            self._finalizer()
        self.dev_ptr = 0

    def __int__(self) -> int:
        return self.dev_ptr
