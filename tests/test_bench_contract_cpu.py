"""The benchmark's reference arm on the host cores: one JSON line with the keys the harness reads.
(The GPU arm needs a B200; its line is checked in the GPU runs.)"""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=REPO)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip().startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    for key in ("metric", "value", "n_gpus", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data",
                "config", "cpu_baseline", "e2e"):
        assert key in d, key
    staged = (REPO / "oracle" / "_ref" / "tree" / ".staged").exists()        # the reference's own code, else the NumPy port
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] == ("reference" if staged else "port") and d["cpu_baseline"]["cores"] == 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"] and "model" not in d["config"] and "rows" in d["config"]


def test_both_arms_name_the_same_workload():
    sys.path.insert(0, str(REPO))
    import bench

    assert bench.WORKLOAD.startswith("configs[1]") and "8192" in bench.METRIC
    w = bench.median_window([3.0, 1.0, 2.0, 10.0, 2.5])
    assert w == {"n": 5, "median_ms": 2.5, "min_ms": 1.0, "max_ms": 10.0}
    named, rest = bench.split_suite([{"kernel": "add_c3_f32"}, {"kernel": "exp_f32"}, {"kernel": "maxpool2d_fwd_c1_f32"}])
    assert [r["kernel"] for r in named] == ["add_c3_f32", "maxpool2d_fwd_c1_f32"] and [r["kernel"] for r in rest] == ["exp_f32"]


def test_reference_arm_is_silent_on_other_ranks():
    env = {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1", "PATH": "/usr/bin:/bin"}
    r = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120, cwd=REPO, env={**__import__("os").environ, **env})
    assert r.returncode == 0 and r.stdout.strip() == ""
