"""ctypes loader for ``libkeydnn_b200.so``.

The role of the reference's ``native_cuda/python/_native_loader.py:37-150`` and
of its per-op ctypes modules (``native_cuda/python/*_ctypes.py``): open the
shared library once per process, give every export its ``argtypes`` and turn a
non-zero status into ``RuntimeError``.  Signatures are read from
``include/keydnn_b200.h`` so the header stays the single description of the ABI.

There is no CPU fallback: a missing library raises ``NativeLibraryError``.
"""
from __future__ import annotations

import ctypes
import os
import re
from functools import lru_cache
from pathlib import Path
from typing import Callable, Dict, List, Tuple

PKG_DIR = Path(__file__).resolve().parent
HEADER_PATH = PKG_DIR.parent / "include" / "keydnn_b200.h"
DEFAULT_LIB_PATH = PKG_DIR / "lib" / "libkeydnn_b200.so"
DNN_HEADER_PATH = PKG_DIR.parent / "include" / "keydnn_b200_dnn.h"
DNN_LIB_PATH = PKG_DIR / "lib" / "libkeydnn_b200_dnn.so"


class NativeLibraryError(RuntimeError):
    """The CUDA operator library is missing or does not export what the header declares."""


_SCALARS = {
    "int": ctypes.c_int,
    "int64_t": ctypes.c_int64,
    "uint64_t": ctypes.c_uint64,
    "size_t": ctypes.c_size_t,
    "float": ctypes.c_float,
    "double": ctypes.c_double,
}

_DECL_RE = re.compile(r"(?:const\s+char\s*\*|int)\s+(keydnn_\w+)\s*\(([^)]*)\)\s*;", re.S)


def parse_header(path: Path = HEADER_PATH) -> Dict[str, Tuple[object, List[object], List[str]]]:
    """Return ``{name: (restype, argtypes, argnames)}`` for every declaration in the header."""
    text = path.read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    out: Dict[str, Tuple[object, List[object], List[str]]] = {}
    for m in _DECL_RE.finditer(text):
        name, args = m.group(1), m.group(2).strip()
        restype = ctypes.c_char_p if m.group(0).lstrip().startswith("const") else ctypes.c_int
        argtypes: List[object] = []
        argnames: List[str] = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a:
                    argtypes.append(ctypes.c_void_p)
                    argnames.append(a.split("*")[-1].strip())
                else:
                    toks = [t for t in a.split(" ") if t != "const"]
                    ctype, pname = toks[0], toks[-1]
                    if ctype not in _SCALARS:
                        raise NativeLibraryError(f"{name}: unknown C type {ctype!r} in {a!r}")
                    argtypes.append(_SCALARS[ctype])
                    argnames.append(pname)
        out[name] = (restype, argtypes, argnames)
    return out


class Native:
    """Handle to the loaded library; ``native.call("keydnn_cuda_add_f32", a, b, y, n)``."""

    def __init__(self, path: Path, strict: bool = True, header: Path = HEADER_PATH):
        self.path = Path(path)
        if not self.path.exists():
            raise NativeLibraryError(
                f"{self.path} not found: build it with `python -m keydnn_v2_b200.build` "
                "(there is no CPU fallback for the CUDA path)"
            )
        self.lib = ctypes.CDLL(str(self.path))
        self.signatures = parse_header(header)
        self._fn: Dict[str, Callable] = {}
        missing = []
        for name, (restype, argtypes, _) in self.signatures.items():
            try:
                f = getattr(self.lib, name)
            except AttributeError:
                missing.append(name)
                continue
            f.restype = restype
            f.argtypes = argtypes
            self._fn[name] = f
        self.missing = missing
        if missing and strict:
            raise NativeLibraryError(f"{self.path} lacks {len(missing)} declared symbols: {missing[:8]}")

    def raw(self, name: str) -> Callable:
        """The bound foreign function (returns the status, raises nothing)."""
        return self._fn[name]

    def error_string(self, code: int) -> str:
        if "keydnn_cuda_error_string" not in self._fn:
            return "status code"
        s = self._fn["keydnn_cuda_error_string"](int(code))
        return s.decode() if s else "?"

    def call(self, name: str, *args) -> None:
        st = self._fn[name](*args)
        if st != 0:
            raise RuntimeError(f"{name} failed with status {st} ({self.error_string(st)})")

    def has(self, name: str) -> bool:
        return name in self._fn


@lru_cache(maxsize=4)
def _load(path: str) -> Native:
    return Native(Path(path))


@lru_cache(maxsize=1)
def load_dnn() -> Native:
    """The cuBLAS / cuDNN wrapper library (Conv2d, Linear); needs libcudnn / libcublas at load time.

    Its calls are enqueued on the operator library's stream: the address of that library's
    ``keydnn_cuda_get_stream`` is bound here once and asked before every cuDNN / cuBLAS call, so there is
    one stream state for both libraries (``keydnn_cuda_set_stream`` moves both)."""
    dnn = Native(Path(os.environ.get("KEYDNN_B200_DNN_LIB") or DNN_LIB_PATH), header=DNN_HEADER_PATH)
    main = load()
    getter = ctypes.cast(main.raw("keydnn_cuda_get_stream"), ctypes.c_void_p).value
    dnn.call("keydnn_dnn_bind_stream_source", getter)
    return dnn


def load(path: str | os.PathLike | None = None) -> Native:
    """Load (once) and return the library.  ``KEYDNN_B200_LIB`` overrides the in-tree path."""
    p = path or os.environ.get("KEYDNN_B200_LIB") or DEFAULT_LIB_PATH
    return _load(str(p))
