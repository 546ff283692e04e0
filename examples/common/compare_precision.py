"""Compares two precision-checker dump directories (the ``.npy`` tensors written with
``--precision_check "level=...,save_tensors=true,path=..."``) tensor by tensor.

    python examples/common/compare_precision.py run_a/ run_b/ [--atol 1e-5] [--rtol 1e-3]

Files are matched by their path relative to each root (rank directory / context / name_count.npy).
A pair passes when ``numpy.allclose(a, b, atol, rtol)``, the tolerance of the reference's own
comparison (scripts/precision_check/precision_compare.py:68,77-78); the first tensor that differs is
usually where two runs start to diverge.  Exit status 1 when anything differs or is missing.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np


def _index(root: str):
    out = {}
    for base, _, files in os.walk(root):
        for f in files:
            if f.endswith(".npy"):
                full = os.path.join(base, f)
                out[os.path.relpath(full, root)] = full
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("a")
    ap.add_argument("b")
    ap.add_argument("--atol", type=float, default=1e-5)
    ap.add_argument("--rtol", type=float, default=1e-3)
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args(argv)
    ia, ib = _index(args.a), _index(args.b)
    bad = 0
    for rel in sorted(set(ia) | set(ib)):
        if rel not in ia or rel not in ib:
            print(f"[MISSING] {rel} in {'first' if rel not in ia else 'second'} run")
            bad += 1
            continue
        x, y = np.load(ia[rel]), np.load(ib[rel])
        if x.shape != y.shape:
            print(f"[SHAPE]   {rel}: {x.shape} vs {y.shape}")
            bad += 1
            continue
        if np.allclose(x, y, atol=args.atol, rtol=args.rtol, equal_nan=True):
            if args.verbose:
                print(f"[ok]      {rel}")
            continue
        diff = np.abs(x.astype(np.float64) - y.astype(np.float64))
        denom = np.maximum(np.abs(y.astype(np.float64)), 1e-12)
        print(f"[DIFF]    {rel}: max abs {diff.max():.3e}, max rel {(diff / denom).max():.3e}, "
              f"{int((diff > args.atol + args.rtol * np.abs(y)).sum())} of {x.size} elements out of tolerance")
        bad += 1
    print(f"{len(set(ia) & set(ib))} tensors compared, {bad} problems")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
