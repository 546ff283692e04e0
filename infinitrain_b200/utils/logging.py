"""Logging and the per-step metric line.

The step line is byte-compatible with the reference's (example/gpt2/main.cc:489-497) so that its
``compare_loss.py`` / ``compare_tps.py`` parse this framework's logs unchanged; a second, optional
line carries the device-timed figures the reference does not have.
"""
from __future__ import annotations

import datetime
import sys


def _stamp(level: str) -> str:
    now = datetime.datetime.now()
    return f"{level}{now:%Y%m%d %H:%M:%S.%f} "


def LOG(level: str, msg: str, file=None) -> None:
    print(_stamp(level[0].upper()) + msg, file=file or sys.stderr, flush=True)


def format_step_line(step: int, num_iteration: int, loss: float, lr: float, duration_ms: float, tps: float,
                     peak_used_mb: float, peak_reserved_mb: float, dp: int, tp: int, sp: int, pp: int) -> str:
    return (f"step {step:4d}/{num_iteration} | train loss {loss:.6f} | lr {lr:.2e} | ({duration_ms:.2f} ms | "
            f"{tps:.0f} tok/s | peak used: {peak_used_mb:5.0f} MB | peak reserved: {peak_reserved_mb:5.0f} MB, "
            f"DP={dp}, TP={tp}, SP={sp}, PP={pp})")


class MetricsSink:
    """Appends one JSON object per step to a file (``.jsonl``): step, loss, learning rate, host- and
    device-timed step time, tokens/s, peak memory, topology.  The reference only has the text line."""

    def __init__(self, path: str):
        import os

        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        self._f = open(path, "a", buffering=1)

    def write(self, **record) -> None:
        import json
        import time

        record.setdefault("time", time.time())
        self._f.write(json.dumps(record) + "\n")

    def close(self) -> None:
        self._f.close()
