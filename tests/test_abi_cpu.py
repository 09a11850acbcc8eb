"""CPU-only checks of the drop-in boundary: the library builds for sm_100a, loads without a GPU,
exports every symbol the header declares and every hot-path symbol the reference's own CUDA
library exports (tests/golden/reference_cuda_exports.txt: `nm -D` of the reference sources
compiled unmodified by oracle/build.py).  No compute call is made here."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib_path():
    from keydnn_v2_b200.build import build_native

    return build_native()


def _exports(path) -> set[str]:
    out = subprocess.check_output(["nm", "-D", "--defined-only", str(path)], text=True)
    return {ln.split()[-1] for ln in out.splitlines() if " T " in ln}


def test_library_exports_every_declared_symbol(lib_path):
    from keydnn_v2_b200._native import parse_header

    declared = set(parse_header())
    exported = {s for s in _exports(lib_path) if s.startswith("keydnn_")}
    assert len(declared) > 140
    assert declared - exported == set()
    assert exported - declared == set(), "every export must be declared in include/keydnn_b200.h"


def test_library_covers_the_reference_hot_path_exports(lib_path):
    want = set((REPO / "tests" / "golden" / "reference_cuda_exports.txt").read_text().split())
    assert len(want) >= 100
    assert want - _exports(lib_path) == set()


def test_library_loads_and_binds_without_a_gpu(lib_path):
    from keydnn_v2_b200 import load

    n = load()
    assert n.raw("keydnn_b200_abi_version")() == 1
    assert n.raw("keydnn_cuda_add_f32").argtypes == [ctypes.c_void_p] * 3 + [ctypes.c_int64]
    assert n.raw("keydnn_cuda_mul_f32").argtypes[-1] is ctypes.c_int            # reference ABI: int numel
    assert n.raw("keydnn_cuda_gt_scalar_f64").argtypes[1] is ctypes.c_double


def test_missing_library_fails_loudly(tmp_path):
    from keydnn_v2_b200._native import Native, NativeLibraryError

    with pytest.raises(NativeLibraryError):
        Native(tmp_path / "libkeydnn_b200.so")


def test_product_package_never_imports_the_oracle():
    for py in (REPO / "keydnn_v2_b200").glob("*.py"):
        text = py.read_text()
        assert "oracle" not in text.replace("# oracle", ""), f"{py.name} mentions the oracle"
