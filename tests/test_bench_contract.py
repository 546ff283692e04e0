"""bench.py's command-line contract as far as it can be checked without a GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    """On a machine that cannot run the reference (no GPU driver) the arm reports itself unavailable
    in one JSON line; where it can, the line carries the metric."""
    r = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=1800, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference"
    assert ("unavailable" in rec and isinstance(rec["unavailable"], str)) or rec["value"] > 0


def test_llama_reference_arm_reports_itself_unavailable_without_a_gpu():
    """The LLaMA-3 arm (a streamed random-init llm.c weight file fed to the reference's stock trainer)
    writes nothing on a machine whose CUDA driver is absent."""
    r = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--model", "llama3-8b", "--tp", "8"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    rec = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][0])
    assert r.returncode == 0 and "unavailable" in rec


@pytest.mark.gpu
def test_bench_line_has_the_contract_keys():
    r = subprocess.run([sys.executable, "bench.py", "--steps", "3", "--warmup", "3"], capture_output=True, text=True,
                       timeout=1200, cwd=ROOT, env={**os.environ, "ITB_NO_REBUILD": "1"})
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in rec, key
    assert rec["n_gpus"] == 1 and rec["steps"] == 3 and rec["value"] > 0 and rec["gpu_launches"] > 0
    assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(rec["e2e"])
    assert {"model", "global_batch", "seq_len", "parallelism"} <= set(rec["config"])
