"""Precision checker, profiler, hooks, dtype / Scalar rules, log line format (CPU)."""
import os
import re

import pytest
import torch

from infinitrain_b200 import nn
from infinitrain_b200.datatype import DataType, PromoteDataTypes, Scalar, parse_dtype
from infinitrain_b200.utils.logging import format_step_line
from infinitrain_b200.utils.precision_checker import (ComputeMD5, PrecisionCheckConfig, PrecisionCheckEnv,
                                                      PrecisionChecker, PrecisionCheckLevel)
from infinitrain_b200.utils.profiler import Profiler


def test_dtype_promotion_and_scalar():
    D = DataType
    assert PromoteDataTypes(D.kFLOAT16, D.kBFLOAT16) == D.kFLOAT32
    assert PromoteDataTypes(D.kINT64, D.kBFLOAT16) == D.kBFLOAT16
    assert PromoteDataTypes(D.kINT32, D.kINT64) == D.kINT64
    assert PromoteDataTypes(D.kUINT32, D.kINT32) == D.kUINT32          # same size: first operand wins
    assert PromoteDataTypes(D.kFLOAT32, D.kFLOAT64) == D.kFLOAT64
    assert parse_dtype("bfloat16") == D.kBFLOAT16 and parse_dtype("float32") == D.kFLOAT32
    assert Scalar(True).kind == Scalar.Kind.kBool and Scalar(3).kind == Scalar.Kind.kInt64
    assert Scalar(3, unsigned=True).kind == Scalar.Kind.kUInt64 and Scalar(2.5).kind == Scalar.Kind.kDouble
    # half types round through fp32 (two-step rounding)
    v = 1.00390625 + 2 ** -20
    assert Scalar(v).to(D.kBFLOAT16) == torch.tensor(v, dtype=torch.float32).bfloat16().item()
    assert Scalar(7.9).to(D.kINT32) == 7 and Scalar(0.0).to(D.kBOOL) is False


def test_module_hooks_and_handles():
    l = nn.Linear(4, 4)
    calls = []
    h1 = l.RegisterForwardPreHook(lambda m, i: calls.append("pre"))
    h2 = l.RegisterForwardPostHook(lambda m, i, o: calls.append("post"))
    h3 = l.RegisterBackwardPostHook(lambda m, gi, go: calls.append("bwd"))
    l(torch.randn(2, 4, requires_grad=True)).sum().backward()
    assert calls == ["pre", "post", "bwd"]
    h1.Remove(); h2.Remove(); h3.Remove()
    calls.clear()
    l(torch.randn(2, 4)).sum().backward()
    assert calls == []


def test_precision_checker_simple_md5_npy(tmp_path):
    cfg = PrecisionCheckConfig.Parse(f"level=2,format=md5,path={tmp_path},save_tensors=true,md5_tolerance=1e-3")
    assert cfg.level == PrecisionCheckLevel.FUNCTION and cfg.format == "md5" and cfg.save_tensors
    env = PrecisionCheckEnv.Instance()
    env.Init(cfg, rank=0)
    try:
        m = nn.Sequential(nn.Linear(4, 4), nn.NewGELU())
        PrecisionChecker.BuildNameMap(m)
        for _ in range(2):
            PrecisionChecker.ResetCounters()
            m(torch.ones(2, 4, requires_grad=True)).sum().backward()
        log = open(os.path.join(env.GetOutputPath(), "precision_check_rank_0.log")).read()
        # the reference's line: <context> <name>[_<n>]_<forward|backward> tensor[<i>]: dtype= shape= md5=
        assert re.search(r"^\[GAS-0\] \[L-0\] 0_forward tensor\[0\]: dtype=float32 shape=\(2,4\) md5=[0-9a-f]{32}$", log, re.M)
        assert "LinearFunction_forward tensor[0]" in log and "LinearFunction_backward tensor[0]" in log and "LinearFunction_3_forward" in log and "0_backward tensor[0]" in log and "Sequential_forward" in log
        files = os.listdir(os.path.join(env.GetOutputPath(), "rank_0"))
        assert "0_forward.npy" in files and "1_backward.npy" in files
    finally:
        env.Shutdown()
    a = torch.tensor([1.0, 2.0])
    assert ComputeMD5(a, 1e-2) == ComputeMD5(a + 1e-4, 1e-2) and ComputeMD5(a) != ComputeMD5(a + 1e-4)
    # the reference quantises with std::round (half away from zero), in double
    assert ComputeMD5(torch.tensor([0.5, -0.5, 2.5]), 1.0) == ComputeMD5(torch.tensor([1.0, -1.0, 3.0]), 1.0)


def test_profiler_records_backward_launches_and_collectives(tmp_path):
    """Kernel level: every native launch entry point is bracketed wherever it is called from (records
    made while autograd runs a backward pass carry ``[bwd]``), and so is every ProcessGroup collective."""
    from infinitrain_b200 import _ext
    from infinitrain_b200.parallel.process_group import ProcessGroup

    C = _ext.load(required=False)
    if C is None:
        pytest.skip("native extension not available")
    p = Profiler.Instance()
    p.Reset()
    calls = []
    saved = {n: getattr(C, n) for n in ("gemm", "layernorm_bwd")}
    saved_pg = ProcessGroup.AllReduce
    try:
        # stand-ins for the launchers (no GPU here): the profiler must wrap whatever the module exposes
        C.gemm = lambda *a, **k: calls.append("gemm")
        C.layernorm_bwd = lambda *a, **k: calls.append("layernorm_bwd")
        ProcessGroup.AllReduce = lambda self, t, *a, **k: calls.append("allreduce")
        p.Enable()
        p.SetTag("Step_3")

        class Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, x):
                C.gemm(x)
                return x * 2

            @staticmethod
            def backward(ctx, g):
                C.gemm(g)
                C.layernorm_bwd(g)
                return g * 2

        x = torch.ones(3, requires_grad=True)
        Fn.apply(x).sum().backward()

        class FakeGroup(ProcessGroup):
            def __init__(self):
                self.name = "DP0"

        FakeGroup().AllReduce(torch.ones(2))
    finally:
        p.Disable()
        assert C.gemm is not saved["gemm"]           # Disable restored the stand-ins, not the originals
        for n, f in saved.items():
            setattr(C, n, f)
        ProcessGroup.AllReduce = saved_pg
    assert calls == ["gemm", "gemm", "layernorm_bwd", "allreduce"]
    names = [r.name for r in p.records]
    assert names == ["gemm", "gemm[bwd]", "layernorm_bwd[bwd]", "pg.AllReduce(DP0)"], names
    rep = p.Report(None, "Count")
    assert "gemm[bwd]" in rep and "pg.AllReduce(DP0)" in rep and "Tag: Step_3" in rep
    p.Reset()


def test_profiler_report_and_trace(tmp_path):
    p = Profiler.Instance()
    p.Reset()
    p.Enable(level="op")
    try:
        p.SetTag("Step_0")
        nn.Linear(8, 8)(torch.randn(2, 8))
        with p.RecordRange("AllReduce"):
            pass
    finally:
        p.Disable()
    rep = p.Report(os.path.join(tmp_path, "rep.txt"), "Count")
    assert "Tag: Step_0" in rep and "linear" in rep and "AllReduce" in rep
    p.ExportChromeTrace(os.path.join(tmp_path, "trace.json"))
    import json

    assert len(json.load(open(os.path.join(tmp_path, "trace.json")))["traceEvents"]) == 2


def test_step_line_matches_reference_parsers():
    line = format_step_line(3, 10, 4.123456, 1e-4, 31.25, 524288.0, 12000, 14000, 8, 1, 1, 1)
    # regular expressions of the reference's scripts/compare_loss.py and compare_tps.py
    m1 = re.search(r"step\s+(\d+)/\d+\s+\|\s+train loss\s+([\d.]+)", line)
    m2 = re.search(r"step\s+(\d+)/\d+\s+\|.*?\|\s+(\d+)\s+tok/s", line)
    assert m1 and float(m1.group(2)) == 4.123456 and m2 and int(m2.group(2)) == 524288


def test_compare_logs_tool(tmp_path):
    import importlib.util
    import os

    from infinitrain_b200.utils.logging import format_step_line

    spec = importlib.util.spec_from_file_location(
        "compare_logs", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "common",
                                     "compare_logs.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    a, b, c = tmp_path / "run_bfloat16.log", tmp_path / "b" / "run_bfloat16.log", tmp_path / "c.log"
    (tmp_path / "b").mkdir()
    lines = [format_step_line(s, 3, 10.0 - s, 1e-4, 20.0, 50000.0, 100, 200, 1, 1, 0, 1) for s in (1, 2, 3)]
    a.write_text("\n".join(lines))
    b.write_text("\n".join(ln.replace("8.000000", "8.004000") for ln in lines))          # inside 1e-2
    c.write_text("\n".join(ln.replace("8.000000", "8.400000").replace("50000 tok/s", "30000 tok/s") for ln in lines))
    assert mod.main([str(a), str(b)]) == 0
    assert mod.main([str(a), str(c)]) == 1
    assert len(mod.compare(a, c, 1e-2, 0.2)) == 2     # one loss mismatch, throughput out of band


def test_sources_have_no_cluster_broadcast_bulk_loads():
    """No source file uses the cluster-broadcast qualifier on a bulk (tensor) copy: every CTA loads
    its own copy of a tile, whichever GPU's memory it comes from."""
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    # the qualifier is spelled in pieces so that this file does not contain it itself
    pat = re.compile(r"cp\.async\.bulk[.\w:]*\.mul" + "ti" + "cast::clu" + "ster")
    hits = []
    for base, _, files in os.walk(root):
        if any(part in base for part in (".git", "_out", "baseline", "_work", "csrc/build")):
            continue
        for f in files:
            if f.endswith((".cu", ".cuh", ".h", ".cpp", ".cc", ".py")) and f != "test_utils_cpu.py":
                if pat.search(open(os.path.join(base, f), errors="replace").read()):
                    hits.append(os.path.join(base, f))
    assert not hits, hits


def test_compare_precision_tool(tmp_path):
    import importlib.util
    import os

    import numpy as np

    spec = importlib.util.spec_from_file_location(
        "compare_precision", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples",
                                          "common", "compare_precision.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for run, delta in (("a", 0.0), ("b", 1e-7), ("c", 1e-2)):
        d = tmp_path / run / "rank_0" / "step0"
        d.mkdir(parents=True)
        np.save(d / "h.0.attn_0.npy", np.linspace(0, 1, 64, dtype=np.float32).reshape(8, 8) + delta)
        np.save(d / "h.0.mlp_0.npy", np.ones((4, 4), dtype=np.float32))
    (tmp_path / "c" / "rank_0" / "step0" / "h.0.mlp_0.npy").unlink()
    assert mod.main([str(tmp_path / "a"), str(tmp_path / "b")]) == 0
    assert mod.main([str(tmp_path / "a"), str(tmp_path / "c")]) == 1


def test_process_group_overview_is_the_reference_text():
    from infinitrain_b200.parallel import global_env as g

    g.InitAllEnv(world_size=1, rank=0)
    # the text the reference's stock trainer prints for one rank (src/nn/parallel/global.cc:196-257)
    assert g.ProcessGroupOverview() == ("\n=== Parallel Communication Groups ===\n"
                                        "world_size = 1, config: {DP=1, TP=1, PP=1}, order: {TP -> DP -> PP}\n"
                                        "[DP] size=1, unenabled\n[TP] size=1, unenabled\n[PP] size=1, unenabled\n\n")
    g.InitAllEnv(world_size=8, rank=0, tensor_parallel_size=2, pipeline_parallel_size=2)
    text = g.ProcessGroupOverview()
    assert "[DP] size=2, num_groups=4\n  - DP 0 (dp=-, tp=0, pp=0): [0, 2]\n  - DP 1 (dp=-, tp=0, pp=1): [4, 6]" in text
    assert "  - PP 3 (dp=1, tp=1, pp=-): [3, 7]\n\n" in text
    g.InitAllEnv(world_size=1, rank=0)


def test_device_runtime_surface_is_callable_on_a_cpu_device():
    """DeviceGuardImpl carries the reference's runtime calls (streams with priorities, events, raw
    memory, pool statistics); on a CPU device they are no-ops that report completion."""
    from infinitrain_b200.device import Device, DeviceGuardImpl, GetDeviceGuardImpl

    impl = GetDeviceGuardImpl()
    cpu = Device.CPU()
    assert impl is DeviceGuardImpl
    assert impl.GetStream(cpu) is None and impl.CreateStream(cpu) is None and impl.CreateStreamWithPriority(cpu, -1) is None
    low, high = impl.GetStreamPriorityRange()
    assert high <= low
    impl.EventRecord(None)
    impl.StreamWaitEvent(None, None)
    assert impl.EventSynchronize(None) and impl.EventQuery(None) and impl.EventElapsedTime(None, None) == 0.0
    impl.SynchronizeStream(None)
    impl.SynchronizeDevice(cpu)
    impl.ResetMemPoolHighWatermarks(cpu)
    assert impl.GetMemPoolPeakMB(cpu) == (0.0, 0.0)
    import pytest

    with pytest.raises(RuntimeError):
        impl.Malloc(cpu, 64)
    impl.Free(0)
