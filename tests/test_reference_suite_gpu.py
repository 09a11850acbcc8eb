"""The reference's own Python stack and its own tests, run against this repository's library.

`oracle/build.py::stage_reference_tree` lays the reference's package and the CUDA-facing part of its
test-suite out under `oracle/_ref/tree/` (git-ignored; staged where a checkout of the reference exists and
shipped from there).  Nothing of the reference is edited: `keydnn_v2_b200.dropin.place` links
`libkeydnn_b200_dropin.so` at the path the reference's loader hard-codes
(`native_cuda/python/_native_loader.py:79-90`), `dropin.install_shim` supplies `ctypes.windll` /
`os.add_dll_directory` on Linux, and the reference's tests are run with pytest in a child process exactly as
they are written: its ctypes bindings (both styles: attribute lookup with `argtypes`, and `GetProcAddress`),
its `_CudaStorage`, Tensor dispatch, autograd closures and pooling Functions all call into this library.

The reference library's exports this repository does not provide (`conv2d_transpose`, `stack`: out of scope,
GAN / RNN models only) are excluded by file name; everything else in the staged directories runs.

Control: a test of the reference that fails here is run once more against the reference's OWN library
(`oracle/_ref/libkeydnn_ref_cuda_full.so`: every `.cu` of its DLL compiled unmodified).  If it fails there as
well it is a defect of that test (or something the reference does not support on this platform), it is
reported and does not count; a test that passes on the reference's library and fails on this one is a
boundary bug and fails the run.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
TREE = REPO / "oracle" / "_ref" / "tree"
REF_FULL = REPO / "oracle" / "_ref" / "libkeydnn_ref_cuda_full.so"

CONFTEST = '''\
"""Written by tests/test_reference_suite_gpu.py of the B200 library: loader shim for Linux, nothing else."""
import sys
sys.path.insert(0, {repo!r})
from keydnn_v2_b200 import dropin
dropin.install_shim()
'''

# raw ctypes bindings (the boundary itself), then the ops / ext layer, Tensor level with autograd, pooling Functions / Modules
GROUPS = {
    "ctypes": ["tests/infrastructure/native_cuda"],
    "ops": ["tests/infrastructure/ops", "tests/infrastructure/reduce"],
    "tensor": ["tests/infrastructure/tensors/cuda"],
    "pool2d": ["tests/infrastructure/pool2d"],
    # whole-stack: Linear / Conv2d Functions and Modules, model training and saving on the CUDA path, the XOR
    # CPU-vs-CUDA gradient parity, activations / losses / optimizers, the remaining Tensor tests
    "stack": ["tests/infrastructure/linear", "tests/infrastructure/conv2d", "tests/infrastructure/models",
              "tests/infrastructure/dropout", "tests/infrastructure/flatten", "tests/infrastructure/tensors/test_*.py",
              "tests/infrastructure/test_xor_grad_parity_f32_cpu_vs_cuda.py", "tests/infrastructure/test_parameter.py",
              "tests/infrastructure/test_activations.py", "tests/infrastructure/test_losses.py",
              "tests/infrastructure/test_optimizers.py", "tests/infrastructure/test_function.py",
              "tests/infrastructure/test_exp.py"],
}
# exports of the reference DLL that are out of scope here
OUT_OF_SCOPE = ("conv2d_transpose", "stack")


def run_reference_tests(paths, lib=None):
    """Runs the reference's tests under `paths` (directories or test ids, relative to the staged tree) against
    `lib` (default: this repository's drop-in library); returns (counts, ids of failed tests, output tail)."""
    from keydnn_v2_b200 import dropin

    dropin.place(TREE / "src" / "keydnn", lib=lib)
    (TREE / "conftest.py").write_text(CONFTEST.format(repo=str(REPO)))
    deselect = " and ".join(f"not {w}" for w in OUT_OF_SCOPE)
    paths = [q for p in paths for q in (sorted(str(f.relative_to(TREE)) for f in TREE.glob(p)) if "*" in p else [p])]
    cmd = [sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--maxfail=1000", "-k", deselect, "--no-header",
           "-rfE", *paths]
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    env.pop("PYTEST_CURRENT_TEST", None)
    r = subprocess.run(cmd, cwd=TREE, capture_output=True, text=True, env=env, timeout=1500)
    tail = (r.stdout + r.stderr)[-6000:]
    counts = {k: 0 for k in ("passed", "failed", "skipped", "error", "errors")}
    summary = [ln for ln in r.stdout.splitlines() if re.search(r"\d+ (passed|failed|skipped|error)", ln)]
    if summary:
        for n, what in re.findall(r"(\d+) (passed|failed|skipped|errors|error)", summary[-1]):
            counts[what] = int(n)
    counts["error"] += counts.pop("errors")
    failed = [m.group(1) for m in (re.match(r"(?:FAILED|ERROR) (\S+)", ln) for ln in r.stdout.splitlines()) if m]
    return counts, failed, tail


@pytest.mark.gpu
@pytest.mark.parametrize("group", list(GROUPS))
def test_reference_tests_pass_against_this_library(group):
    if not (TREE / ".staged").exists():
        pytest.skip("no staged copy of the reference (oracle/build.py::stage_reference_tree needs a checkout of it)")
    try:
        counts, failed, tail = run_reference_tests(GROUPS[group])
        also_on_reference = []
        if failed and REF_FULL.exists():
            # control: the same tests against the reference's own library
            _, failed_there, _ = run_reference_tests(failed, lib=REF_FULL)
            also_on_reference = [t for t in failed if t in failed_there]
    finally:
        from keydnn_v2_b200 import dropin

        dropin.place(TREE / "src" / "keydnn")          # leave this repository's library in place
    ours_only = [t for t in failed if t not in also_on_reference]
    print(f"reference tests [{group}]: {counts}; failing on the reference's own library as well: {also_on_reference}; "
          f"failing on this library only: {ours_only}")
    (REPO / "gpurun_out").mkdir(exist_ok=True)
    with open(REPO / "gpurun_out" / "reference_suite_counts.txt", "a") as f:
        f.write(f"{group}: {counts} fails_on_reference_too={also_on_reference} fails_here_only={ours_only}\n")
    assert not ours_only, tail
    assert counts["passed"] > 0, tail


def test_reference_loader_opens_the_drop_in_library_without_a_gpu():
    """No device call: the reference's unmodified loader finds the library at its hard-coded path, and both of
    its binding styles resolve symbols of both libraries behind the umbrella."""
    if not (TREE / ".staged").exists():
        pytest.skip("no staged copy of the reference")
    from keydnn_v2_b200 import dropin

    dropin.place(TREE / "src" / "keydnn")
    code = f"""
import sys
sys.path.insert(0, {str(REPO)!r}); sys.path.insert(0, {str(TREE)!r})
from keydnn_v2_b200 import dropin
dropin.install_shim()
from src.keydnn.infrastructure.native_cuda.python._native_loader import load_keydnn_cuda_native
from src.keydnn.infrastructure.native_cuda.python.ops import tensor_arithmetic_ctypes as ta
lib = load_keydnn_cuda_native()
assert lib.keydnn_b200_dropin_version() == 1
for name in ("keydnn_cuda_add_f32", "keydnn_cuda_maxpool2d_forward_f32", "keydnn_cuda_sum_all_f64",
             "keydnn_cuda_matmul_f32", "keydnn_cuda_conv2d_forward_f32"):
    assert getattr(lib, name) is not None and ta._get_proc_addr(lib, name) != 0, name
print("drop-in ok")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "drop-in ok" in r.stdout, r.stdout + r.stderr
