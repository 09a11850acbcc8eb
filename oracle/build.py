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
* ``stage_reference_tree(ref_root)`` - lays out, under ``oracle/_ref/tree/``, the reference's Python package
  (``src/keydnn``, ``*.py`` only) and the CUDA-facing part of its test-suite (``tests/infrastructure/...``) so that
  the reference's own bindings, Tensor code and tests can be run against this repository's library on a
  machine that has no checkout of the reference (``tests/test_reference_suite_gpu.py``), and so that the
  benchmark's reference arm can time the reference's own CPU Tensor methods.  Like the compiled objects, the
  staged tree exists only in ``oracle/_ref/`` (git-ignored, never committed): nothing of it enters the history.
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
REF_NATIVE_OMP = REF_DIR / "libkeydnn_ref_native_omp.so"     # all four CPU kernels files, OpenMP build
REF_CUDA_FULL = REF_DIR / "libkeydnn_ref_cuda_full.so"       # every .cu of the reference DLL (links cuBLAS / cuDNN)

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
# A checkout of the reference project: the KEYDNN_REFERENCE_ROOT environment variable, else the sibling
# directory `reference` of this repository (where the build container mounts it).  Absent on other machines.
DEFAULT_REF_ROOT = Path(os.environ.get("KEYDNN_REFERENCE_ROOT") or HERE.parent.parent / "reference")
REF_TREE = REF_DIR / "tree"
# the reference's test directories that exercise its CUDA library (relative to tests/infrastructure)
REF_TEST_DIRS = ["native_cuda", "tensors", "ops", "reduce", "pool2d", "linear", "conv2d", "models", "dropout", "flatten"]
# ... and single files of tests/infrastructure that train whole models on the CUDA path
REF_TEST_FILES = ["test_xor_grad_parity_f32_cpu_vs_cuda.py", "test_parameter.py", "test_activations.py", "test_losses.py",
                  "test_optimizers.py", "test_function.py", "test_exp.py"]
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
    # the library the reference's CPU ops load (pooling + its OpenMP convolutions), built as its Linux script
    # builds the OpenMP variant (scripts/_build_native_linux.sh:79-110)
    all_cpps = [nat / f for f in ("keydnn_maxpool2d.cpp", "keydnn_avgpool2d.cpp", "keydnn_conv2d.cpp",
                                  "keydnn_conv2d_transpose.cpp")]
    if force or not REF_NATIVE_OMP.exists():
        _run(["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-I", str(nat), *map(str, all_cpps), "-o",
              str(REF_NATIVE_OMP)])
    out["native_omp"] = REF_NATIVE_OMP
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cus = [ref_root / REF_CUDA_SUBDIR / f for f in REF_CUDA_SOURCES]
    if force or not REF_CUDA.exists():
        _run([nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
              "-shared", "-w", *map(str, cus), "-o", str(REF_CUDA)])
    out["cuda"] = REF_CUDA
    # the whole reference DLL (matmul / conv2d / conv2d_transpose / stack included): the control when one of the
    # reference's own tests fails against this repository's library - does it pass against the reference's?
    all_cus = sorted((ref_root / REF_CUDA_SUBDIR).glob("*.cu"))
    if force or not REF_CUDA_FULL.exists():
        try:
            _run([nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
                  "-shared", "-w", *map(str, all_cus), "-o", str(REF_CUDA_FULL), "-lcublas", "-lcudnn"])
        except RuntimeError as exc:     # optional: needs the cuBLAS / cuDNN development files
            print(f"reference DLL with cuBLAS / cuDNN not built: {str(exc)[:300]}", file=sys.stderr)
    if REF_CUDA_FULL.exists():
        out["cuda_full"] = REF_CUDA_FULL
    return out


def stage_reference_tree(ref_root: str | Path | None = None, force: bool = False) -> Path | None:
    """``oracle/_ref/tree/{src/keydnn, tests/infrastructure/...}`` from a checkout of the reference; None without one."""
    ref_root = Path(ref_root) if ref_root is not None else DEFAULT_REF_ROOT
    if not (ref_root / "src" / "keydnn").exists():
        return REF_TREE if REF_TREE.exists() else None
    stamp = REF_TREE / ".staged"
    if stamp.exists() and not force:
        return REF_TREE
    if REF_TREE.exists():
        shutil.rmtree(REF_TREE)
    keep_py = shutil.ignore_patterns("__pycache__", "*.pyc", "*.cu", "*.cuh", "*.hpp", "*.h", "*.cpp", "*.dll", "*.so",
                                     "*.vcxproj*", "*.sln", "*.lib", "*.exp", "*.pdb", "x64")
    shutil.copytree(ref_root / "src" / "keydnn", REF_TREE / "src" / "keydnn", ignore=keep_py)
    (REF_TREE / "src" / "__init__.py").touch()
    tests_src, tests_dst = ref_root / "tests", REF_TREE / "tests"
    (tests_dst / "infrastructure").mkdir(parents=True)
    for init in (tests_src / "__init__.py", tests_src / "infrastructure" / "__init__.py"):
        if init.exists():
            shutil.copy(init, tests_dst / init.relative_to(tests_src))
    for d in REF_TEST_DIRS:
        if (tests_src / "infrastructure" / d).exists():
            shutil.copytree(tests_src / "infrastructure" / d, tests_dst / "infrastructure" / d, ignore=keep_py)
            parent = (tests_dst / "infrastructure" / d).parent
            src_init = tests_src / "infrastructure" / Path(d).parent / "__init__.py"
            if parent != tests_dst / "infrastructure" and src_init.exists():
                shutil.copy(src_init, parent / "__init__.py")
    for f in REF_TEST_FILES:
        if (tests_src / "infrastructure" / f).exists():
            shutil.copy(tests_src / "infrastructure" / f, tests_dst / "infrastructure" / f)
    # the reference's CPU pooling kernels where its loader looks for them (native/python/_native_loader.py:110-117)
    if REF_NATIVE_OMP.exists():
        shutil.copy(REF_NATIVE_OMP, REF_TREE / "src" / "keydnn" / "infrastructure" / "native" / "python" / "libkeydnn_native_omp.so")
    for path in [REF_TREE, *REF_TREE.rglob("*")]:        # a read-only checkout hands down read-only modes
        path.chmod(path.stat().st_mode | 0o200)
    stamp.write_text("staged from a checkout of the reference; not part of this repository\n")
    return REF_TREE


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
    print(stage_reference_tree(force="--force" in sys.argv))
