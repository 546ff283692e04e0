"""Profiler: per-kernel host / device time and peak memory, per-tag reports, NVTX ranges and a
Chrome-trace export.

Reference: infini_train/src/profiler.cc:41-313 and include/dispatcher.h:22-43 (compile-time
PROFILE_MODE; every dispatched kernel, forward and backward, is bracketed by stream synchronisation,
device time from events, mem-pool peak; per-rank report and record files; collectives are not seen).
Here profiling is a runtime switch.  ``Profiler.Instance().Enable()`` brackets

* every launch entry point of the native extension (``gemm``, ``flash_attn_fwd / _bwd``,
  ``layernorm_fwd / _bwd``, ``adamw``, ..., and the fused NVLink kernels ``tp_gemm``,
  ``nvl_allreduce_scale``, ``nvl_rs_adamw_bcast``, ``nvl_ce_merge``), whoever calls it -- the forward
  wrappers, the ``autograd.Function.backward``s (records made while autograd runs a backward pass are
  named ``<entry>[bwd]``), the optimizers, the reducer;
* every collective of ``ProcessGroup`` (``AllReduce``, ``AllGather``, ``ReduceScatter``, ``Send``,
  ``Recv``, ``BroadCast``, ``Barrier``), named ``pg.<Collective>(<group>)``;

each with a host time, a device time (events on the stream the launch goes to, so kernels on the
communication side stream are timed there) and an NVTX range.  ``Enable(level="op")`` records the
ten fused forward ops as units instead (their inner launches are then nested and not listed).
Records carry the current tag (``SetTag("Step_9")``); ``Report`` prints the reference's table (count,
host us, device us, averages, peak MB) sortable by seven keys; ``ExportChromeTrace`` writes a timeline
the reference cannot produce.  Like the reference's profile build, an enabled profiler serialises
the step: its numbers are shares, not a benchmark.
"""
from __future__ import annotations

import json
import time
from collections import defaultdict
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass
class ProfileRecord:
    tag: str
    name: str
    device: str
    host_us: float
    device_us: float
    peak_mem_mb: float
    start_us: float


class Profiler:
    _instance = None
    SortKeys = ("HostTimeTotal", "HostTimeAverage", "DeviceTimeTotal", "DeviceTimeAverage", "Count", "PeakMemory",
                "NotSorted")

    def __init__(self):
        self.enabled = False
        self.records: List[ProfileRecord] = []
        self.tag = "Untagged"
        self.depth = 0
        self.level = "kernel"
        self._orig = []
        self._t0 = time.perf_counter()

    @classmethod
    def Instance(cls) -> "Profiler":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def SetTag(self, tag: str):
        self.tag = tag

    # ------------------------------------------------------------------ recording
    @contextmanager
    def RecordRange(self, name: str, device: Optional[torch.device] = None):
        """Times ``name`` on the host and (on CUDA) on the device; nested ranges are ignored like
        nested kernel calls in the reference.  Also pushes an NVTX range."""
        if not self.enabled or self.depth > 0:
            self.depth += 1
            try:
                yield
            finally:
                self.depth -= 1
            return
        self.depth += 1
        cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        if cuda:
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_push(name)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            host_us = (time.perf_counter() - t0) * 1e6
            dev_us, peak = 0.0, 0.0
            if cuda:
                e1.record()
                e1.synchronize()
                dev_us = e0.elapsed_time(e1) * 1e3
                torch.cuda.nvtx.range_pop()
                peak = torch.cuda.max_memory_reserved() / (1 << 20)
            self.records.append(ProfileRecord(self.tag, name, "cuda" if cuda else "cpu", host_us, dev_us, peak,
                                              (t0 - self._t0) * 1e6))
            self.depth -= 1

    # entry points of the native extension that launch kernels (everything else in the module is a
    # query or a mode switch)
    kNativeLaunchers = ("gemm", "layernorm_fwd", "layernorm_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "gelu_fwd", "gelu_bwd",
                        "swiglu_fwd", "swiglu_bwd", "rope_inplace", "embedding_fwd", "embedding_bwd", "ce_fwd", "ce_bwd",
                        "adamw", "adam_advance", "sgd", "cast_into", "colsum", "flash_attn_fwd", "flash_attn_bwd",
                        "nvl_allreduce_scale", "nvl_rs_adamw_bcast", "nvl_ce_merge", "tp_gemm", "tp_wait")
    kCollectives = ("AllReduce", "AllGather", "ReduceScatter", "Send", "Recv", "BroadCast", "Barrier")
    kForwardOps = ("linear", "mlp_gelu", "layernorm", "rmsnorm", "gelu", "swiglu", "swiglu_packed", "attention_packed",
                   "embedding", "cross_entropy")

    @staticmethod
    def _in_backward() -> bool:
        try:
            return torch._C._current_graph_task_id() != -1
        except Exception:  # noqa: BLE001
            return False

    def _wrap(self, owner, attr: str, label):
        orig = getattr(owner, attr)
        self._orig.append((owner, attr, orig))

        def wrapped(*a, _orig=orig, **k):
            name = label(a) if callable(label) else label
            if self._in_backward():
                name += "[bwd]"
            with self.RecordRange(name):
                return _orig(*a, **k)

        setattr(owner, attr, wrapped)

    def Enable(self, level: str = "kernel"):
        """``level="kernel"`` (default): every native launch and every collective is a record.
        ``level="op"``: the fused forward ops are the records (what they launch inside is nested)."""
        from .. import _ext
        from ..ops import functional as ops
        from ..parallel.process_group import ProcessGroup

        if self.enabled:
            return
        if level not in ("kernel", "op"):
            raise ValueError("profiler level must be 'kernel' or 'op'")
        self.enabled = True
        self.level = level
        self._orig = []
        if level == "op":
            for fname in self.kForwardOps:
                self._wrap(ops, fname, fname)
        C = _ext.load(required=False)
        if C is not None:
            for fname in self.kNativeLaunchers:
                if hasattr(C, fname):
                    self._wrap(C, fname, fname)
        for cname in self.kCollectives:
            if hasattr(ProcessGroup, cname):
                self._wrap(ProcessGroup, cname,
                           lambda a, _c=cname: f"pg.{_c}({getattr(a[0], 'name', '?')})" if a else f"pg.{_c}")

    def Disable(self):
        for owner, attr, orig in reversed(self._orig):
            setattr(owner, attr, orig)
        self._orig = []
        self.enabled = False

    def Reset(self):
        self.records.clear()

    # ------------------------------------------------------------------ reports
    def Aggregate(self, tag: Optional[str] = None) -> Dict[str, dict]:
        agg = defaultdict(lambda: dict(count=0, host_us=0.0, device_us=0.0, peak_mb=0.0))
        for r in self.records:
            if tag is not None and r.tag != tag:
                continue
            a = agg[r.name]
            a["count"] += 1
            a["host_us"] += r.host_us
            a["device_us"] += r.device_us
            a["peak_mb"] = max(a["peak_mb"], r.peak_mem_mb)
        return dict(agg)

    def Report(self, path: Optional[str] = None, sort_by: str = "DeviceTimeTotal") -> str:
        keyfn = {"HostTimeTotal": lambda kv: -kv[1]["host_us"],
                 "HostTimeAverage": lambda kv: -kv[1]["host_us"] / kv[1]["count"],
                 "DeviceTimeTotal": lambda kv: -kv[1]["device_us"],
                 "DeviceTimeAverage": lambda kv: -kv[1]["device_us"] / kv[1]["count"],
                 "Count": lambda kv: -kv[1]["count"], "PeakMemory": lambda kv: -kv[1]["peak_mb"],
                 "NotSorted": lambda kv: 0}[sort_by]
        lines = []
        for tag in sorted({r.tag for r in self.records}):
            agg = self.Aggregate(tag)
            tot = sum(a["device_us"] for a in agg.values()) or 1.0
            lines.append(f"Tag: {tag}")
            lines.append(f"{'Name':<24}{'Count':>8}{'Host Total(us)':>16}{'Host Avg(us)':>14}{'Device Total(us)':>18}"
                         f"{'Device Avg(us)':>16}{'Device %':>10}{'Peak Mem(MB)':>14}")
            for name, a in sorted(agg.items(), key=keyfn):
                lines.append(f"{name:<24}{a['count']:>8}{a['host_us']:>16.2f}{a['host_us'] / a['count']:>14.2f}"
                             f"{a['device_us']:>18.2f}{a['device_us'] / a['count']:>16.2f}"
                             f"{100 * a['device_us'] / tot:>9.2f}%{a['peak_mb']:>14.1f}")
            lines.append("")
        text = "\n".join(lines)
        if path:
            with open(path, "w") as f:
                f.write(text)
        return text

    def PrintRecords(self, path: str) -> None:
        with open(path, "w") as f:
            for r in self.records:
                f.write(f"{r.tag}\t{r.name}\t{r.device}\thost_us={r.host_us:.2f}\tdevice_us={r.device_us:.2f}"
                        f"\tpeak_mb={r.peak_mem_mb:.1f}\n")

    def ExportChromeTrace(self, path: str, rank: int = 0) -> None:
        ev = [{"name": r.name, "cat": r.tag, "ph": "X", "ts": r.start_us, "dur": max(r.device_us, r.host_us),
               "pid": rank, "tid": 0, "args": {"host_us": r.host_us, "device_us": r.device_us}} for r in self.records]
        with open(path, "w") as f:
            json.dump({"traceEvents": ev, "displayTimeUnit": "ms"}, f)
