"""Shared fixtures.  GPU tests carry ``@pytest.mark.gpu`` and call the CUDA library
through its C ABI; everything else runs on a CPU-only machine."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parents[1]
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference's own CPU path (see tests/golden/make_golden.py)."""
    with np.load(REPO / "tests" / "golden" / "ref_cpu_golden.npz") as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def oracle():
    from oracle import build as ob
    from oracle import keydnn_oracle

    ob.build_oracle()
    return keydnn_oracle


@pytest.fixture(autouse=True)
def _guard_bands_intact(request):
    """GPU tests: every `tests/_gpu_util.Buf` released during the test must have both guard bands intact."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import gc

    import _gpu_util

    gc.collect()
    found, _gpu_util.OVERRUNS[:] = list(_gpu_util.OVERRUNS), []
    assert not found, found
