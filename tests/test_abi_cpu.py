"""CPU-only checks of the drop-in boundary: the library builds for sm_100a, loads without a GPU,
exports every symbol the header declares and every hot-path symbol the reference's own CUDA
library exports (tests/golden/reference_cuda_exports.txt: `nm -D` of the reference sources
compiled unmodified by oracle/build.py).  No compute call is made here."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
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


def test_dnn_library_exports_every_declared_symbol():
    from keydnn_v2_b200._native import DNN_HEADER_PATH, parse_header
    from keydnn_v2_b200.build import build_dnn

    declared = set(parse_header(DNN_HEADER_PATH))
    exported = {s for s in _exports(build_dnn()) if s.startswith("keydnn_")}
    assert declared - exported == set()
    assert exported - declared == set(), "every export must be declared in include/keydnn_b200_dnn.h"


def test_both_libraries_share_one_stream_state(lib_path):
    """The cuDNN / cuBLAS library has no stream of its own once loaded through the package: it asks the operator
    library before every call, so `keydnn_cuda_set_stream` moves both (no device call is made here: the stream
    values are only stored and read back)."""
    from keydnn_v2_b200 import load
    from keydnn_v2_b200._native import load_dnn

    lib, dnn = load(), load_dnn()
    seen = ctypes.c_uint64(1)
    try:
        for value in (0xABC0, 0x1230, 0):
            lib.call("keydnn_cuda_set_stream", value)
            dnn.call("keydnn_dnn_get_stream", ctypes.byref(seen))
            assert seen.value == value
    finally:
        lib.call("keydnn_cuda_set_stream", 0)


def test_column_reduction_chunk_arithmetic_is_64_bit(lib_path):
    """Narrow matrices with close to 2^31 rows: rows per chunk and the chunk count come out of 64-bit
    arithmetic, and a shape whose last chunk would reach past 2^31 - 1 is refused (-2) instead of
    wrapping around.  Host arithmetic only, nothing is allocated or launched."""
    from keydnn_v2_b200 import load

    f = load().raw("keydnn_cuda_debug_col_chunks")
    out = (ctypes.c_int64 * 3)()
    for rows in (1, 31, 32, 33, 4096, 8192, 1 << 20, (1 << 30) + 7, (1 << 31) - 4096):
        for cols, esz in ((8, 4), (1024, 4), (4096, 8)):
            st = f(rows, cols, esz, 8, out)
            assert st == 0, (rows, cols, esz)
            rch, nchunks, stripes = out
            assert rch > 0 and rch % 8 == 0 and 1 <= nchunks <= 65535 and stripes >= 1
            assert (nchunks - 1) * rch < rows <= nchunks * rch
            assert nchunks * rch + 32 <= 2**31 - 1
    assert f(2**31 - 1, 8, 4, 8, out) == -2         # the last chunk would end beyond INT_MAX
    assert f(0, 8, 4, 8, out) == -2


def test_pool_band_plans_fit_their_shared_memory(lib_path):
    """The split of a plane into row bands, for two thousand seeded geometries and both element sizes: the bands cover
    the plane, the dynamic shared memory stays under the 48 KiB a launch gets without opting in, and every region the
    kernels index (staging buffers with up to one packet of alignment slack, the quotient rows with their extra column
    and row, the row table) fits - with the number of output rows that cover a band counted by brute force, not by
    the bound the planner uses.  Host arithmetic only, nothing is allocated or launched."""
    from keydnn_v2_b200 import load

    f = load().raw("keydnn_cuda_debug_pool_band_plan")
    out = (ctypes.c_int64 * 5)()
    rng = np.random.default_rng(11)
    usable = 0
    for _ in range(2000):
        H, W = int(rng.integers(1, 600)), int(rng.integers(1, 2500))
        k = (int(rng.integers(1, 8)), int(rng.integers(1, 8)))
        s = (int(rng.integers(1, 6)), int(rng.integers(1, 6)))
        p = (int(rng.integers(0, k[0] // 2 + 1)), int(rng.integers(0, k[1] // 2 + 1)))
        if H + 2 * p[0] < k[0] or W + 2 * p[1] < k[1]:
            continue
        Ho, Wo = (H + 2 * p[0] - k[0]) // s[0] + 1, (W + 2 * p[1] - k[1]) // s[1] + 1
        for esz in (4, 8):
            vec = 16 // esz
            for kind in (0, 1, 2):
                assert f(kind, esz, H, W, Ho, Wo, k[0], k[1], s[0], s[1], p[0], p[1], out) == 0
                ok, rows, bands, smem, buf = out
                if not ok:
                    continue
                usable += 1
                extent = Ho if kind == 0 else H
                assert rows >= 1 and bands >= 1 and rows * (bands - 1) < extent <= rows * bands
                assert smem <= 48 * 1024, (kind, esz, H, W, k, s, p, smem)
                if kind == 0:
                    span = ((rows - 1) * s[0] + k[0]) * W                 # input elements a band can stage
                    assert buf % vec == 0 and buf >= span + vec - 1 and smem >= 2 * buf * esz
                    continue
                covering = 0                                            # most output rows that cover one band
                for b in range(bands):
                    h0, h1 = b * rows, min(H, (b + 1) * rows)
                    lo = max(0, -(-(h0 + p[0] - k[0] + 1) // s[0]))
                    hi = min(Ho - 1, (h1 - 1 + p[0]) // s[0])
                    covering = max(covering, hi - lo + 1)
                staged = (covering + 1) * (Wo + 1)
                arrive = covering * Wo + (vec if kind == 1 else 4) - 1
                assert buf >= arrive, (kind, esz, H, W, k, s, p)
                if kind == 1:
                    assert smem >= rows * 8 + staged * esz + 2 * buf * esz
                else:
                    assert smem >= rows * 16 + staged * (esz + 4) + 2 * buf * (esz + 8)
    assert usable > 3000


def test_every_reference_signature_is_declared_with_the_same_argument_classes():
    """All argument lists, not a sample: tests/golden/reference_cuda_signatures.json holds the argument list of every
    `keydnn_*` function of the reference's CUDA library reduced to register classes (pointer, 32 / 64-bit integer,
    float, double; made by tests/golden/make_signatures.py from its .hpp / .cu text).  Every one this repository
    declares - in either header - must have exactly that list."""
    import json

    from keydnn_v2_b200._native import DNN_HEADER_PATH, parse_header

    ref = json.loads((REPO / "tests" / "golden" / "reference_cuda_signatures.json").read_text())
    ours = {**parse_header(), **parse_header(DNN_HEADER_PATH)}
    classes = {ctypes.c_void_p: "ptr", ctypes.c_int: "i32", ctypes.c_int64: "i64", ctypes.c_uint64: "u64",
               ctypes.c_size_t: "u64", ctypes.c_float: "f32", ctypes.c_double: "f64"}
    hot_path = set((REPO / "tests" / "golden" / "reference_cuda_exports.txt").read_text().split())
    checked, wrong = 0, {}
    for name, want in ref.items():
        if name not in ours:
            assert name not in hot_path, f"{name} is a hot-path export of the reference and is not declared here"
            continue                      # out of scope (conv2d_transpose, stack, debug helpers)
        got = [classes[t] for t in ours[name][1]]
        checked += 1
        if got != want:
            wrong[name] = (got, want)
    assert not wrong, wrong
    assert checked >= len(hot_path) and hot_path <= set(ours)
