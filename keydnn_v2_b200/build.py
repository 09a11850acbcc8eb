"""Build the sm_100a shared libraries in-tree with nvcc.

`python -m keydnn_v2_b200.build` compiles every `csrc/*.cu` into
`keydnn_v2_b200/lib/libkeydnn_b200.so`.  nvcc cross-compiles without a GPU, so
the build also runs on a CPU-only machine; the built library is loaded with
`ctypes` by `keydnn_v2_b200._native`.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libkeydnn_b200.so"
DNN_SRC = PKG_DIR / "csrc_dnn" / "dnn.cu"
DNN_LIB_PATH = LIB_DIR / "libkeydnn_b200_dnn.so"
DROPIN_SRC = PKG_DIR / "csrc_dropin" / "dropin.c"
DROPIN_LIB_PATH = LIB_DIR / "libkeydnn_b200_dropin.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-fmad=false",          # every product/sum rounds on its own, as in the reference build
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set NVCC or put /usr/local/cuda/bin on PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


# translation units that keep nvcc's default FMA contraction: their transcendental functions must
# expand exactly as in the reference build; their own arithmetic uses explicitly rounded intrinsics
DEFAULT_FMAD = {"activation.cu", "softmax.cu"}


def _compile(src: Path, verbose: bool, extra: list[str]) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    if _newer(obj, [src, *headers, Path(__file__)]):
        return obj
    flags = [f for f in NVCC_FLAGS if not (src.name in DEFAULT_FMAD and f == "-fmad=false")]
    cmd = [_nvcc(), *ARCH_FLAGS, *flags, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, flush=True)
    return obj


def build_native(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile and link the library; returns its path.  Up-to-date objects are kept."""
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose or ptxas_info, extra), srcs))
    if not force and _newer(LIB_PATH, objs):
        return LIB_PATH
    cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-ldl"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


def build_dnn(force: bool = False, verbose: bool = False) -> Path:
    """The cuBLAS / cuDNN wrapper library (Linear and Conv2d stay library calls)."""
    LIB_DIR.mkdir(exist_ok=True)
    if not force and _newer(DNN_LIB_PATH, [DNN_SRC, Path(__file__)]):
        return DNN_LIB_PATH
    cmd = [_nvcc(), *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
           "-fvisibility=hidden", "-shared", str(DNN_SRC), "-o", str(DNN_LIB_PATH), "-lcudnn", "-lcublas"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {DNN_SRC.name}:\n{r.stdout}\n{r.stderr}")
    return DNN_LIB_PATH


def build_dropin(force: bool = False, verbose: bool = False) -> Path:
    """The single file that stands in for the reference's one CUDA DLL: depends on both libraries above (found
    next to it through $ORIGIN) and binds their stream state when it is loaded."""
    if not force and _newer(DROPIN_LIB_PATH, [DROPIN_SRC, LIB_PATH, DNN_LIB_PATH, Path(__file__)]):
        return DROPIN_LIB_PATH
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", str(DROPIN_SRC), "-o", str(DROPIN_LIB_PATH),
           "-L", str(LIB_DIR), "-Wl,--no-as-needed", "-lkeydnn_b200", "-lkeydnn_b200_dnn", "-Wl,-rpath,$ORIGIN"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"gcc failed for {DROPIN_SRC.name}:\n{r.stdout}\n{r.stderr}")
    return DROPIN_LIB_PATH


if __name__ == "__main__":
    print(build_dnn(force="--force" in sys.argv, verbose=True))
    p = build_native(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(p)
    print(build_dropin(force="--force" in sys.argv, verbose=True))
