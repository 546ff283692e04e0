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


def test_secondary_falls_back_to_the_eager_step_and_all_ranks_agree(tmp_path, monkeypatch):
    """The second half of the headline metric runs in child processes after the parents have released
    their communicator.  Stand-in child: the graph attempt fails on rank 1 only; both parents must
    then move on to the eager attempt together, and rank 0 returns that record with the reason."""
    import importlib.util
    import threading
    import types

    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    child = tmp_path / "child.py"
    child.write_text(
        "import json, os, sys\n"
        "graph = sys.argv[sys.argv.index('--graph') + 1]\n"
        "if graph == '1' and os.environ['RANK'] == '1':\n"
        "    sys.stderr.write('capture failed on this rank\\n'); sys.exit(3)\n"
        "if os.environ['RANK'] == '0':\n"
        "    print(json.dumps({'value': 1.0, 'graph': graph, 'port': os.environ['MASTER_PORT']}))\n")
    monkeypatch.setenv("ITB_TEST_ARTIFACTS", str(tmp_path))
    monkeypatch.setenv("MASTER_PORT", "29900")
    args = types.SimpleNamespace(gpus=2, steps=2, warmup=1, layers=0, secondary_budget=120)
    out = {}

    def parent(rank):
        env_rank = {"RANK": str(rank)}
        # each parent hands its own RANK to its child through the environment of the subprocess call
        real_popen = bench.subprocess.Popen

        def popen(cmd, **kw):
            kw["env"] = {**kw["env"], **env_rank}
            return real_popen(cmd, **kw)

        local = types.SimpleNamespace(**{k: getattr(bench.subprocess, k) for k in ("PIPE", "TimeoutExpired")}, Popen=popen)
        out[rank] = bench._run_secondary(args, rank, str(child), local)

    threads = [threading.Thread(target=parent, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert out[1] is None
    rec = out[0]
    assert rec["graph"] == "0" and rec["attempt"] == "eager", rec
    assert "cuda graph: exited with code 3" in rec["earlier_attempts"][0] and "capture failed" in rec["earlier_attempts"][0]
    assert rec["port"] == str(29900 + 13 + 7)
