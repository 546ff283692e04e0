"""Runs the example trainers over a matrix of configurations and keeps one log per run, for
regression checks with ``compare_logs.py``.

    python examples/common/run_matrix.py examples/common/matrix_smoke.json --out logs/
    python examples/common/run_matrix.py my_matrix.json --out logs_new/ --compare logs_old/
    python examples/common/run_matrix.py examples/common/matrix_gpu.json --out logs/ --profile --ctest build/

The last line is the whole regression round on a GPU node in one command, as the reference's
scripts/run_models_and_profile.bash does over scripts/test_config.json: the native suites through ctest
(``--ctest`` names a configured CMake build directory), every configuration once for its loss and
throughput log, once more with the kernel profiler on (``--profile``; reports go to ``<out>/profile``),
then the comparison against an earlier round's logs (``--compare``).  Runs that need more GPUs than the
machine has are skipped and listed.

``--frontend cpp`` runs the same matrix through the C++ trainer (``examples/cpp/train.cc``), which takes the
same flags and prints the same step line.

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


def _cpp_trainer(cuda: bool) -> str:
    """Path of the C++ trainer, built when it is missing or older than its sources."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("itb_cpp_build", os.path.join(ROOT, "examples", "cpp", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return str(mod.build(cuda=cuda))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("matrix")
    ap.add_argument("--out", required=True)
    ap.add_argument("--compare", default="", help="baseline log directory to compare against afterwards")
    ap.add_argument("--only", default="", help="comma-separated run ids")
    ap.add_argument("--port", type=int, default=29700)
    ap.add_argument("--tps-band", type=float, default=0.2, help="throughput tolerance handed to compare_logs.py")
    ap.add_argument("--profile", action="store_true", help="run every configuration a second time with --profile")
    ap.add_argument("--ctest", default="", help="CMake build directory: build it and run its ctest suites first")
    ap.add_argument("--dry-run", action="store_true", help="print the commands without running them")
    ap.add_argument("--frontend", default="python", choices=["python", "cpp"],
                    help="cpp: run the matrix through the C++ trainer (examples/cpp/train.cc, built on demand)")
    args = ap.parse_args(argv)
    spec = json.load(open(args.matrix))
    os.makedirs(args.out, exist_ok=True)
    only = set(filter(None, args.only.split(",")))
    failed, skipped = [], []
    on_gpu = spec.get("common", {}).get("device", "") == "cuda"
    gpus = 0
    if on_gpu:
        import torch

        gpus = torch.cuda.device_count()
    if args.ctest and not args.dry_run:
        label = "cuda" if gpus else "cpu"
        for cmd in (["cmake", "--build", args.ctest, "-j", str(os.cpu_count() or 4)],
                    ["ctest", "--test-dir", args.ctest, "-L", label, "--output-on-failure"]):
            r = subprocess.run(cmd, cwd=ROOT)
            if r.returncode != 0:
                print(f"[FAIL] {' '.join(cmd)}", flush=True)
                failed.append("ctest")
                break
    passes = [("", {})] + ([("profile", {"profile": True})] if args.profile else [])
    todo = [(i, run, p) for p in passes for i, run in enumerate(spec["runs"])]
    for i, run, (pass_name, pass_flags) in todo:
        if only and run["id"] not in only:
            continue
        family, nproc = run.get("family", "gpt2"), int(run.get("nproc", 1))
        if on_gpu and nproc > gpus and not args.dry_run:
            if not pass_name:
                skipped.append(f"{family}_{run['id']} (needs {nproc} GPUs, {gpus} visible)")
            continue
        flags = dict(spec.get("common", {}))
        flags.update(run.get("args", {}))
        flags.update(pass_flags)
        if args.frontend == "cpp":
            cmd = [_cpp_trainer(on_gpu and not args.dry_run), "--family", family, *_flags(flags)]
        else:
            cmd = [sys.executable, os.path.join(ROOT, "examples", family, "main.py"), *_flags(flags)]
        if nproc > 1:
            sys.path.insert(0, ROOT)
            from infinitrain_b200 import _ext

            launcher = _ext.launcher_path()
            if not launcher.exists():
                _ext.build_launcher()
            cmd = [str(launcher), f"--nproc_per_node={nproc}", f"--rdzv_endpoint=127.0.0.1:{args.port + i}", "--", *cmd]
        # the profiler writes its reports into the working directory: one directory per profiled run
        out_dir = os.path.join(args.out, pass_name, f"{family}_{run['id']}") if pass_name else args.out
        os.makedirs(out_dir, exist_ok=True)
        log = os.path.join(out_dir, f"{family}_{run['id']}.log")
        if args.dry_run:
            print(" ".join(cmd), ">", log)
            continue
        env = dict(os.environ)
        if not on_gpu and "OMP_NUM_THREADS" not in env:
            # CPU ranks share the machine's cores: without a cap every rank starts one thread per core
            env["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // nproc))
        with open(log, "w") as f:
            r = subprocess.run(cmd, stdout=f, stderr=subprocess.STDOUT, cwd=out_dir if pass_name else ROOT, env=env)
        print(f"[{'ok' if r.returncode == 0 else 'FAIL'}] {family}_{run['id']} -> {log}", flush=True)
        if r.returncode != 0:
            failed.append(run["id"])
    for sk in skipped:
        print(f"[skipped] {sk}", flush=True)
    rc = 1 if failed else 0
    if args.compare:
        rc |= subprocess.run([sys.executable, os.path.join(ROOT, "examples", "common", "compare_logs.py"), args.compare,
                              args.out, "--tps-band", str(args.tps_band)]).returncode
    return rc


if __name__ == "__main__":
    sys.exit(main())
