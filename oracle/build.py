"""Build recipes for the checker libraries.  TEST INFRASTRUCTURE ONLY.

* ``build_oracle()``  - gcc over ``oracle/pool_oracle.c`` -> ``oracle/lib/libkeydnn_oracle.so``
  (the CPU restatement of the pooling arithmetic).
* ``build_reference(ref_root)`` - compiles the reference's own sources, where they lie in a
  checkout of the reference project, into ``oracle/_ref/``:
    - ``libkeydnn_ref_native.so``: its CPU pooling kernels
      (``src/keydnn/infrastructure/native/src/keydnn_{max,avg}pool2d.cpp``) with the flags of its
      own Linux build script (``scripts/_build_native_linux.sh:74-117``: -O3 -std=c++17 -fPIC -shared);
    - ``libkeydnn_ref_cuda.so``: the hot-path ``.cu`` files of its CUDA library, unmodified,
      for sm_100a (its Visual Studio project sets no architecture).
  No reference source is copied; only the built objects land in ``oracle/_ref/`` (git-ignored).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "lib" / "libkeydnn_oracle.so"
REF_DIR = HERE / "_ref"
REF_NATIVE = REF_DIR / "libkeydnn_ref_native.so"
REF_CUDA = REF_DIR / "libkeydnn_ref_cuda.so"

# hot-path translation units of the reference CUDA library (no cuBLAS / cuDNN needed)
REF_CUDA_SOURCES = [
    "kernel.cu",
    "keydnn_avgpool2d_cuda.cu",
    "keydnn_global_avgpool2d_cuda.cu",
    "keydnn_pad2d_cuda.cu",
    "keydnn_reduce_cuda.cu",
    "keydnn_tensor_arithmetic.cu",
    "keydnn_mul.cu",
    "keydnn_fill_cuda.cu",
    "keydnn_cuda_utils.cu",
    "keydnn_memcpy_d2d.cu",
    "keydnn_cuda_broadcast_to.cu",
    "keydnn_tensor_bias_add.cu",
    "keydnn_transpose2d.cu",
    "keydnn_cuda_exp.cu",
]
# where a checkout of the reference project is looked for when no path is given
DEFAULT_REF_ROOT = Path(os.environ.get("KEYDNN_REFERENCE_ROOT", "/root/reference"))
REF_CUDA_SUBDIR = "src/keydnn/infrastructure/native_cuda/keydnn_v2_cuda_native/KeyDNNV2CudaNative"
REF_NATIVE_SUBDIR = "src/keydnn/infrastructure/native/src"


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "pool_oracle.c"
    if not force and ORACLE_LIB.exists() and ORACLE_LIB.stat().st_mtime >= src.stat().st_mtime:
        return ORACLE_LIB
    ORACLE_LIB.parent.mkdir(exist_ok=True)
    _run(["gcc", "-O2", "-fPIC", "-shared", "-ffp-contract=off", str(src), "-o", str(ORACLE_LIB), "-lm"])
    return ORACLE_LIB


def build_reference(ref_root: str | Path | None = None, force: bool = False) -> dict[str, Path]:
    """Compile the reference's own pooling .cpp and hot-path .cu files into ``oracle/_ref``."""
    ref_root = Path(ref_root) if ref_root is not None else DEFAULT_REF_ROOT
    out: dict[str, Path] = {}
    if not ref_root.exists():
        return out
    REF_DIR.mkdir(exist_ok=True)
    nat = ref_root / REF_NATIVE_SUBDIR
    cpps = [nat / "keydnn_maxpool2d.cpp", nat / "keydnn_avgpool2d.cpp"]
    if force or not REF_NATIVE.exists():
        _run(["g++", "-O3", "-std=c++17", "-fPIC", "-shared", *map(str, cpps), "-o", str(REF_NATIVE)])
    out["native"] = REF_NATIVE
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cus = [ref_root / REF_CUDA_SUBDIR / f for f in REF_CUDA_SOURCES]
    if force or not REF_CUDA.exists():
        _run([nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
              "-shared", "-w", *map(str, cus), "-o", str(REF_CUDA)])
    out["cuda"] = REF_CUDA
    return out


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
