"""Regression check between two training logs (or two directories of logs) written by the example
trainers: per-step loss within an absolute tolerance and mean throughput within a relative band.

    python examples/common/compare_logs.py baseline.log test.log
    python examples/common/compare_logs.py baseline_dir test_dir --loss-tol-bf16 1e-2 --tps-band 0.2

The step line is the one the trainers print (``step N/M | train loss L | lr ... | (T ms | R tok/s | ...``),
which is also the format the reference's own comparison scripts parse (scripts/compare_loss.py:20,
scripts/compare_tps.py:17); tolerances default to theirs: 1e-5 for fp32 logs, 1e-2 for bf16 logs (a
file whose name contains ``bfloat16`` or ``bf16``), +-20 % on mean tok/s with the first step left out.
Exit status 0 when everything matches, 1 otherwise.
"""
from __future__ import annotations

import argparse
import re
import sys
from pathlib import Path
from typing import Dict, List, Tuple

STEP = re.compile(r"step\s+(\d+)/\d+\s+\|\s+train loss\s+([-+0-9.eEnaif]+).*?\|\s*\(\s*([0-9.]+)\s*ms\s*\|\s*([0-9.]+)\s*tok/s")


def parse(path: Path) -> Dict[int, Tuple[float, float, float]]:
    out = {}
    for line in path.read_text(errors="replace").splitlines():
        m = STEP.search(line)
        if m:
            out[int(m.group(1))] = (float(m.group(2)), float(m.group(3)), float(m.group(4)))
    return out


def is_bf16(path: Path) -> bool:
    return "bfloat16" in path.name or "bf16" in path.name


def compare(a: Path, b: Path, tol: float, band: float) -> List[str]:
    la, lb = parse(a), parse(b)
    problems = []
    if not la or not lb:
        return [f"no step lines in {a if not la else b}"]
    for step in sorted(set(la) | set(lb)):
        if step not in la or step not in lb:
            problems.append(f"step {step}: missing in {(a if step not in la else b).name}")
            continue
        d = abs(la[step][0] - lb[step][0])
        if not d <= tol:      # also catches NaN
            problems.append(f"step {step}: loss {la[step][0]:.6f} vs {lb[step][0]:.6f} (diff {d:.2e} > {tol:.0e})")
    ta = [v[2] for s, v in sorted(la.items()) if s > 1]
    tb = [v[2] for s, v in sorted(lb.items()) if s > 1]
    if ta and tb:
        ma, mb = sum(ta) / len(ta), sum(tb) / len(tb)
        if ma > 0 and abs(mb - ma) / ma > band:
            problems.append(f"throughput: {ma:.0f} vs {mb:.0f} tok/s ({100 * (mb - ma) / ma:+.1f} % outside +-{100 * band:.0f} %)")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("baseline", type=Path)
    ap.add_argument("test", type=Path)
    ap.add_argument("--loss-tol-fp32", type=float, default=1e-5)
    ap.add_argument("--loss-tol-bf16", type=float, default=1e-2)
    ap.add_argument("--tps-band", type=float, default=0.2)
    args = ap.parse_args(argv)
    if args.baseline.is_dir():
        names = sorted(p.name for p in args.baseline.glob("*.log"))
        pairs = [(args.baseline / n, args.test / n) for n in names]
    else:
        pairs = [(args.baseline, args.test)]
    bad = 0
    for a, b in pairs:
        if not b.exists():
            print(f"[MISSING] {b}")
            bad += 1
            continue
        tol = args.loss_tol_bf16 if is_bf16(a) else args.loss_tol_fp32
        problems = compare(a, b, tol, args.tps_band)
        print(f"[{'FAIL' if problems else 'ok'}] {a.name}")
        for p in problems:
            print("   ", p)
        bad += bool(problems)
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
