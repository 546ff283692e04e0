"""Runs the example trainers over a matrix of configurations and keeps one log per run, for
regression checks with ``compare_logs.py``.

    python examples/common/run_matrix.py examples/common/matrix_smoke.json --out logs/
    python examples/common/run_matrix.py my_matrix.json --out logs_new/ --compare logs_old/

The matrix file is JSON: ``{"common": {flag: value, ...}, "runs": [{"id": "...", "family": "gpt2" |
"llama3", "nproc": N, "args": {flag: value, ...}}, ...]}``.  A run with ``nproc > 1`` goes through the
``infini_run`` launcher (one process per rank).  Flags are the trainers' own (``--help``); a boolean
``true`` becomes a bare flag.  The log of run ``id`` is ``<out>/<family>_<id>.log`` (ids of bf16 runs
carry ``bfloat16`` so that the comparison picks the bf16 tolerance).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _flags(d):
    out = []
    for k, v in d.items():
        if v is True:
            out.append(f"--{k}")
        elif v is False or v is None:
            continue
        else:
            out += [f"--{k}", str(v)]
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("matrix")
    ap.add_argument("--out", required=True)
    ap.add_argument("--compare", default="", help="baseline log directory to compare against afterwards")
    ap.add_argument("--only", default="", help="comma-separated run ids")
    ap.add_argument("--port", type=int, default=29700)
    ap.add_argument("--tps-band", type=float, default=0.2, help="throughput tolerance handed to compare_logs.py")
    args = ap.parse_args(argv)
    spec = json.load(open(args.matrix))
    os.makedirs(args.out, exist_ok=True)
    only = set(filter(None, args.only.split(",")))
    failed = []
    for i, run in enumerate(spec["runs"]):
        if only and run["id"] not in only:
            continue
        family, nproc = run.get("family", "gpt2"), int(run.get("nproc", 1))
        flags = dict(spec.get("common", {}))
        flags.update(run.get("args", {}))
        cmd = [sys.executable, os.path.join(ROOT, "examples", family, "main.py"), *_flags(flags)]
        if nproc > 1:
            sys.path.insert(0, ROOT)
            from infinitrain_b200 import _ext

            launcher = _ext.launcher_path()
            if not launcher.exists():
                _ext.build_launcher()
            cmd = [str(launcher), f"--nproc_per_node={nproc}", f"--rdzv_endpoint=127.0.0.1:{args.port + i}", "--", *cmd]
        log = os.path.join(args.out, f"{family}_{run['id']}.log")
        with open(log, "w") as f:
            r = subprocess.run(cmd, stdout=f, stderr=subprocess.STDOUT, cwd=ROOT)
        print(f"[{'ok' if r.returncode == 0 else 'FAIL'}] {family}_{run['id']} -> {log}", flush=True)
        if r.returncode != 0:
            failed.append(run["id"])
    rc = 1 if failed else 0
    if args.compare:
        rc |= subprocess.run([sys.executable, os.path.join(ROOT, "examples", "common", "compare_logs.py"), args.compare,
                              args.out, "--tps-band", str(args.tps_band)]).returncode
    return rc


if __name__ == "__main__":
    sys.exit(main())
