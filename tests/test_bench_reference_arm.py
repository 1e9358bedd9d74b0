"""The benchmark's CPU arm runs without a GPU and prints one JSON line with the
keys the measurement contract names."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_contract_line():
    env = dict(os.environ, OMP_NUM_THREADS="1")      # what torchrun exports; the arm must still use every core
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c1",
                           "--steps", "3", "--warmup", "2"],
                          capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["vs_baseline"] is None and d["data"] == "synthetic" and "workload" in d["config"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    base = d["cpu_baseline"]
    assert base["kind"] == "port" and base["value"] == d["value"] and base["cores"] == os.cpu_count()
    assert d["value"] > 0 and d["ms_per_step"] > 0
    # the arm says what it ran: --steps / --warmup are passes over a bounded sample, which the config names, and
    # the step time is marked as extrapolated from the sample to a full step of the workload
    assert d["steps"] == 3 == base["passes"] and d["warmup"] == 2 == base["warmup_passes"]
    cfg = d["config"]
    assert cfg["sample_requests"] == 8 and cfg["sample_pool_blocks"] == 256 and 0 < cfg["sample_blocks"] < cfg["blocks_per_step"]
    assert "extrapolated" in d["ms_per_step_basis"]
    ratio = cfg["blocks_per_step"] / cfg["sample_blocks"]
    assert abs(d["ms_per_step"] - d["ms_per_sample_pass"] * ratio) < 1e-6 * d["ms_per_step"]
    assert "c_openmp" in base


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2"],
                          capture_output=True, text=True, env=env, timeout=300)
    assert proc.returncode == 0 and proc.stdout.strip() == ""
