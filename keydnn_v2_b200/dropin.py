"""Make KeyDNN's own Python stack call this library: the loader-side change, as code.

KeyDNN (``src/keydnn/infrastructure/native_cuda/python/_native_loader.py:37-150``) opens one native
library at a fixed, Windows-shaped path below its package,

    <keydnn>/infrastructure/native_cuda/keydnn_v2_cuda_native/x64/Release/KeyDNNV2CudaNative.dll

and nine of its binding modules resolve symbols with ``ctypes.windll.kernel32.GetProcAddress`` at import
time (``native_cuda/python/ops/tensor_arithmetic_ctypes.py:54-56`` and siblings).  Nothing in KeyDNN is
edited.  Two things are supplied instead:

* ``install_shim()``: on a platform without ``ctypes.windll`` it installs a ``kernel32.GetProcAddress`` that
  is ``dlsym`` and a no-op ``os.add_dll_directory`` (the loader calls it unguarded, ``:121-122,148``).  Call it
  before the first ``keydnn`` import.
* ``place(keydnn_package_dir)``: links ``libkeydnn_b200_dropin.so`` (which pulls in the operator library and
  the cuDNN / cuBLAS library and binds their stream state) at the path above; ``dlopen`` does not care about
  the ``.dll`` suffix.  ``stack_ctypes.py:80-110`` computes the same path, so it is served too.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

from ._native import NativeLibraryError

PKG_DIR = Path(__file__).resolve().parent
DROPIN_LIB_PATH = PKG_DIR / "lib" / "libkeydnn_b200_dropin.so"
DLL_RELATIVE_PATH = Path("infrastructure") / "native_cuda" / "keydnn_v2_cuda_native" / "x64" / "Release" / "KeyDNNV2CudaNative.dll"


class _Kernel32:
    """``GetProcAddress(handle, name)`` with the meaning it has for the reference's call sites: the address of
    an exported symbol of an already loaded library, or NULL."""

    def __init__(self) -> None:
        self._dlsym = ctypes.CDLL(None).dlsym
        self._dlsym.restype = ctypes.c_void_p
        self._dlsym.argtypes = [ctypes.c_void_p, ctypes.c_char_p]

        def GetProcAddress(handle, name):
            return self._dlsym(handle, name)

        # the call sites assign .argtypes / .restype on the function object: a plain function takes those
        self.GetProcAddress = GetProcAddress


class _Windll:
    def __init__(self) -> None:
        self.kernel32 = _Kernel32()


def install_shim() -> None:
    """Idempotent; does nothing on Windows."""
    if not hasattr(ctypes, "windll"):
        ctypes.windll = _Windll()
    if not hasattr(os, "add_dll_directory"):
        os.add_dll_directory = lambda path: None


def place(keydnn_package_dir: str | os.PathLike, lib: str | os.PathLike | None = None) -> Path:
    """Link the drop-in library at the path KeyDNN's loader opens; returns that path."""
    src = Path(lib or os.environ.get("KEYDNN_B200_DROPIN_LIB") or DROPIN_LIB_PATH).resolve()
    if not src.exists():
        raise NativeLibraryError(f"{src} not found: build it with `python -m keydnn_v2_b200.build`")
    dst = Path(keydnn_package_dir) / DLL_RELATIVE_PATH
    dst.parent.mkdir(parents=True, exist_ok=True)
    if dst.is_symlink() or dst.exists():
        if dst.is_symlink() and dst.resolve() == src:
            return dst
        dst.unlink()
    dst.symlink_to(src)
    return dst
