"""Micro-benchmarks of the hot sm_100a kernels on the shapes of the headline models.

    python -m infinitrain_b200.ops.microbench gemm        # tcgen05 GEMM vs torch.matmul (cuBLAS), GPT-2 shapes
    python -m infinitrain_b200.ops.microbench gemm_llama_tp8   # the same for LLaMA-3 8B's per-rank shapes under TP8
    python -m infinitrain_b200.ops.microbench attention   # tcgen05 vs mma.sync flash attention, forward + backward
    python -m infinitrain_b200.ops.microbench profile     # one launch of each, for a profiler capture
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m infinitrain_b200.ops.microbench tp             # fused vs NCCL tensor-parallel linear pair

Every number is CUDA-event time on the launching stream after warm-up, with a buffer larger than L2
written between timed launches.  One JSON line per case.
"""
from __future__ import annotations

import json
import math
import sys

import torch

from .. import _ext


def _timer():
    flush = torch.empty(64 << 20, device="cuda", dtype=torch.float32)   # 256 MB > 126 MB of L2

    def timeit(fn, n=10, warm=3):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    return timeit


def _attn_tensors(B, T, H, KV, D):
    qkv = torch.randn(B, T, (H + 2 * KV) * D, device="cuda").bfloat16()
    q = qkv[..., : H * D].view(B, T, H, D)
    k = qkv[..., H * D: (H + KV) * D].view(B, T, KV, D)
    v = qkv[..., (H + KV) * D:].view(B, T, KV, D)
    dqkv = torch.empty_like(qkv)
    dq = dqkv[..., : H * D].view(B, T, H, D)
    dk = dqkv[..., H * D: (H + KV) * D].view(B, T, KV, D)
    dv = dqkv[..., (H + KV) * D:].view(B, T, KV, D)
    return q, k, v, dq, dk, dv


def bench_gemm(C, tokens=16 * 1024, layers=((2304, 768), (768, 768), (3072, 768), (768, 3072), (50304, 768))):
    """Forward, input-gradient and weight-gradient GEMM of each linear layer ``(out, in)`` on ``tokens``
    rows.  Defaults: GPT-2 124M at 16 x 1024 tokens."""
    timeit = _timer()
    shapes = []
    for n, k in layers:
        shapes += [("fwd", tokens, n, k), ("dgrad", tokens, k, n), ("wgrad", n, k, tokens)]
    for kind, M, N, K in shapes:
        if kind == "fwd":
            a = torch.randn(M, K, device="cuda").bfloat16()
            b = torch.randn(N, K, device="cuda").bfloat16()
            c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            ours = timeit(lambda: C.gemm(a, False, b, False, M, N, K, c, None, None, None, None, 0, 0))
            lib = timeit(lambda: torch.matmul(a, b.t(), out=c))
        elif kind == "dgrad":
            a = torch.randn(M, K, device="cuda").bfloat16()
            b = torch.randn(K, N, device="cuda").bfloat16()
            c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            ours = timeit(lambda: C.gemm(a, False, b, True, M, N, K, c, None, None, None, None, 0, 0))
            lib = timeit(lambda: torch.matmul(a, b, out=c))
        else:
            a = torch.randn(K, M, device="cuda").bfloat16()
            b = torch.randn(K, N, device="cuda").bfloat16()
            c = torch.zeros(M, N, device="cuda")
            cb = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            ours = timeit(lambda: C.gemm(a, True, b, True, M, N, K, c, None, None, None, None,
                                         C.GEMM_OUT_F32 | C.GEMM_ATOMIC, 0))
            lib = timeit(lambda: torch.matmul(a.t(), b, out=cb))
        fl = 2.0 * M * N * K
        print(json.dumps({"case": "gemm", "kind": kind, "M": M, "N": N, "K": K, "ours_ms": ours, "cublas_ms": lib,
                          "ours_tflops": fl / ours / 1e9, "cublas_tflops": fl / lib / 1e9}))


def bench_gemm_llama_tp8(C):
    """The per-rank GEMMs of LLaMA-3 8B under 8-way tensor parallelism at 1 x 2048 tokens (the skinny
    shapes behind the fused all-gather+GEMM / GEMM+reduce-scatter kernels), without the collectives."""
    bench_gemm(C, tokens=2048, layers=((768, 4096), (4096, 512), (1792, 4096), (4096, 1792), (16032, 4096)))


def bench_gemm_probe(C):
    """Where the CTA-pair GEMM's main loop spends its time: the full kernel against the same launch
    without operand loads (tensor-core issue + shared-memory reads alone) and without MMAs (TMA fill
    of the ring alone).  The probe launches compute nothing meaningful; only their times are read."""
    timeit = _timer()
    for M, N, K in ((8192, 8192, 8192), (16384, 2304, 768), (2048, 16032, 4096)):
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        res = {"case": "gemm_probe", "M": M, "N": N, "K": K}
        probes = (("full", 0), ("no_load", C.GEMM_PROBE_NO_LOAD), ("no_mma", C.GEMM_PROBE_NO_MMA),
                  ("neither", C.GEMM_PROBE_NO_LOAD | C.GEMM_PROBE_NO_MMA))
        for name, fl in probes:
            t = timeit(lambda: C.gemm(a, False, b, False, M, N, K, c, None, None, None, None, fl, 0))
            res[name + "_us"] = t * 1e3
        res["cublas_us"] = timeit(lambda: torch.matmul(a, b.t(), out=c)) * 1e3
        # per k-block of 64 and CTA pair, in SM cycles at the nominal 1.965 GHz
        kblocks = ((M + 255) // 256) * ((N + 255) // 256) * (K // 64) / 74.0
        for name, _ in probes:
            res[name + "_cycles_per_kblock"] = res[name + "_us"] * 1965.0 / kblocks
        res["status"] = C.kernel_status()
        print(json.dumps(res))


def bench_norm(C):
    """LayerNorm / RMSNorm forward and backward on the activations of the headline models, against the
    bytes they have to move (bf16 x, dy in, y / dx out) at the measured copy bandwidth."""
    timeit = _timer()
    for rows, Cd, rms in ((16384, 768, False), (2048, 4096, True), (16384, 4096, True)):
        x = torch.randn(rows, Cd, device="cuda").bfloat16()
        g = torch.ones(Cd, device="cuda")
        b = torch.zeros(Cd, device="cuda")
        dy = torch.randn_like(x)
        dres = torch.randn_like(x)
        res = {"case": "norm", "rows": rows, "C": Cd, "rms": rms}
        if rms:
            y, rstd = C.rmsnorm_fwd(x, g, 1e-5, torch.bfloat16)
            res["fwd_us"] = timeit(lambda: C.rmsnorm_fwd(x, g, 1e-5, torch.bfloat16)) * 1e3
            res["bwd_us"] = timeit(lambda: C.rmsnorm_bwd(dy, x, g, rstd)) * 1e3
            res["bwd_res_us"] = timeit(lambda: C.rmsnorm_bwd(dy, x, g, rstd, dres, None, None, True)) * 1e3
        else:
            y, mean, rstd = C.layernorm_fwd(x, g, b, 1e-5, torch.bfloat16)
            res["fwd_us"] = timeit(lambda: C.layernorm_fwd(x, g, b, 1e-5, torch.bfloat16)) * 1e3
            res["bwd_us"] = timeit(lambda: C.layernorm_bwd(dy, x, g, mean, rstd, True)) * 1e3
            res["bwd_res_us"] = timeit(lambda: C.layernorm_bwd(dy, x, g, mean, rstd, True, dres, None, None, None, True)) * 1e3
        nbytes = rows * Cd * 2
        res["fwd_floor_us"] = 2 * nbytes / 6.5389e12 * 1e6
        res["bwd_floor_us"] = 3 * nbytes / 6.5389e12 * 1e6
        res["bwd_res_floor_us"] = 4 * nbytes / 6.5389e12 * 1e6
        print(json.dumps(res))


def bench_attention(C):
    timeit = _timer()
    default = C.get_attn_mode()
    for B, T, H, KV, D in ((16, 1024, 12, 12, 64), (1, 2048, 32, 8, 128), (4, 2048, 32, 8, 128), (1, 2048, 4, 1, 128)):
        q, k, v, dq, dk, dv = _attn_tensors(B, T, H, KV, D)
        sc = 1.0 / math.sqrt(D)
        o, lse = C.flash_attn_fwd(q, k, v, sc, True)
        do = torch.randn_like(o)
        fl = 4.0 * B * H * T * T * D / 2
        res = {"case": "attention", "B": B, "T": T, "H": H, "KV": KV, "D": D}
        for mode, name in ((0, "mma_sync"), (3, "tcgen05")):
            C.set_attn_mode(mode)
            t = timeit(lambda: C.flash_attn_fwd(q, k, v, sc, True))
            res[f"fwd_{name}_ms"], res[f"fwd_{name}_tflops"] = t, fl / t / 1e9
            t = timeit(lambda: C.flash_attn_bwd(do, q, k, v, o, lse, dq, dk, dv, sc, True))
            res[f"bwd_{name}_ms"], res[f"bwd_{name}_tflops"] = t, 2.5 * fl / t / 1e9
        C.set_attn_mode(default)
        res["status"] = C.kernel_status()
        print(json.dumps(res))


def profile_case(C):
    """GEMM forward (twice) and weight gradient on 16384 x 2304 x 768, attention forward and backward on
    16 x 1024 x 12 heads x 64: the launches a profiler capture of the top kernels needs, and no more."""
    M, N, K = 16384, 2304, 768
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        C.gemm(a, False, b, False, M, N, K, c, None, None, None, None, 0, 0)
    dw = torch.zeros(N, K, device="cuda")
    C.gemm(c, True, a, True, N, K, M, dw, None, None, None, None, C.GEMM_OUT_F32 | C.GEMM_ATOMIC, 0)
    q, k, v, dq, dk, dv = _attn_tensors(16, 1024, 12, 12, 64)
    o, lse = C.flash_attn_fwd(q, k, v, 0.125, True)
    C.flash_attn_bwd(torch.randn_like(o), q, k, v, o, lse, dq, dk, dv, 0.125, True)
    torch.cuda.synchronize()
    print(json.dumps({"case": "profile", "status": C.kernel_status()}))


def bench_tp(C):
    """Column-parallel + row-parallel linear pair (forward + backward) under sequence parallelism on
    every rank of the job: fused all-gather+GEMM / GEMM+reduce-scatter launches against the NCCL
    formulation of the same layers.  Shapes from the environment: TPB_B, TPB_T, TPB_H, TPB_F."""
    import os

    import torch.distributed as dist

    from ..autocast import AutocastGuard
    from ..datatype import DataType
    from ..device import DeviceType
    from ..parallel import global_env as genv
    from ..parallel import symm
    from ..parallel.process_group import ProcessGroupFactory
    from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    genv.InitAllEnv(world_size=world, rank=rank, tensor_parallel_size=world, sequence_parallel_enabled=True)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    B, T = int(os.environ.get("TPB_B", 1)), int(os.environ.get("TPB_T", 2048))
    H, F = int(os.environ.get("TPB_H", 4096)), int(os.environ.get("TPB_F", 28672))
    Tl = T // world
    col = ColumnParallelLinear(H, F, bias=False, gather_output=False, input_is_parallel=False,
                               sequence_parallel=True, device=dev)
    row = RowParallelLinear(F, H, bias=False, input_is_parallel=True, sequence_parallel=True, device=dev)
    for p in list(col.Parameters()) + list(row.Parameters()):
        p.data.normal_(0, 0.02)
        p.main_grad = torch.zeros_like(p)
    x = (torch.randn(B, Tl, H, device=dev) * 0.5).bfloat16().requires_grad_(True)
    res = (torch.randn(B, Tl, H, device=dev) * 0.5).bfloat16()
    gy = torch.randn(B, Tl, H, device=dev).bfloat16() * 0.1
    out = {"case": "tp", "B": B, "T": T, "H": H, "F": F, "world": world}

    def step():
        with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16):
            y = row(col(x), residual=res)
        y.backward(gy)

    for fused in ("0", "1"):
        os.environ["ITB_FUSED_TP"] = fused
        symm.reset_fused_tp()
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = 20
        e0.record()
        for _ in range(n):
            step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["fused_ms" if fused == "1" else "nccl_ms"] = t.item()
    if symm._TP_CTX is not None:
        out["status"] = symm._TP_CTX.nvl.status()
    flops = 3 * 2.0 * B * T * H * (F // world) * 2
    out["fused_tflops_per_gpu"] = flops / out["fused_ms"] / 1e9
    out["nccl_tflops_per_gpu"] = flops / out["nccl_ms"] / 1e9
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


def bench_collectives(C):
    """The data-parallel collectives as NVLink kernels against their NCCL formulation, on every rank
    of the job, per bucket size (25 MB: a DDP bucket; 154 MB: GPT-2's tied embedding bucket):
      * all-reduce(avg) of an fp32 gradient bucket  vs  ncclAllReduce;
      * reduce-scatter + AdamW + broadcast of fp32 weights and bf16 shadows in ONE kernel  vs
        ncclReduceScatter + the AdamW kernel on the shard + ncclAllGather of fp32 weights and of bf16 shadows.
    CUDA events on the launching stream, max over ranks.  The roofline of each is the bytes one GPU has
    to send (= receive) over NVLink divided by the measured peer-copy bandwidth (770 GB/s per direction)."""
    import os
    from types import SimpleNamespace

    import torch.distributed as dist

    from ..parallel import global_env as genv
    from ..parallel import symm
    from ..parallel.process_group import ProcessGroupFactory, dp_group

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    genv.InitAllEnv(world_size=world, rank=rank)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    pg = dp_group()
    ctx = symm.NvlinkContext.get(pg, dev)
    link = 770e9

    def timed(fn, n=20, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for mb in (25, 154):
        n = mb * 1024 * 1024 // 4 // (world * 128) * (world * 128)
        grads = ctx.alloc(n, torch.float32)
        params = ctx.alloc(n, torch.float32)
        shadow = ctx.alloc(n, torch.bfloat16)
        grads.normal_()
        params.normal_()
        res = {"case": "collectives", "world": world, "bucket_mb": mb, "multimem": bool(ctx.ptrs(grads)[1])}
        ar = symm.BucketAllReduce(ctx, grads)
        res["allreduce_fused_ms"] = timed(lambda: ar(grads).WaitNonBlocking())
        res["allreduce_nccl_ms"] = timed(lambda: dist.all_reduce(grads, op=dist.ReduceOp.AVG))
        wire = 4.0 * n * (world - 1) / world          # bytes out of (and into) one GPU
        res["allreduce_floor_ms"] = wire / link * 1e3
        res["allreduce_fraction_of_link"] = res["allreduce_floor_ms"] / res["allreduce_fused_ms"]
        # ZeRO step of the bucket
        shard = n // world
        m, v = torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
        buffer = SimpleNamespace(grad_buffer=grads, param_buffer=params, shadow_buffer=shadow)
        bucket = SimpleNamespace(offset=0, numel=n)
        step = symm.FusedZeroBucketStep(ctx, buffer, bucket, m, v)
        res["zero_fused_ms"] = timed(lambda: step(1e-4, 0.9, 0.999, 1e-8, 0.1, 0.1, 0.001, 1.0 / world).WaitNonBlocking())
        gs = torch.empty(shard, device=dev)
        m2, v2 = torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
        my_p = params[rank * shard:(rank + 1) * shard]
        my_s = shadow[rank * shard:(rank + 1) * shard]

        def nccl_step():
            dist.reduce_scatter_tensor(gs, grads, op=dist.ReduceOp.AVG)
            C.adamw(my_p, gs, m2, v2, my_s, 1e-4, 0.9, 0.999, 1e-8, 0.1, 0.1, 0.001, 1.0, None)
            dist.all_gather_into_tensor(params, my_p)
            dist.all_gather_into_tensor(shadow, my_s)

        res["zero_nccl_ms"] = timed(nccl_step)
        # in: (W-1)/W of the gradients; out: this rank's shard of weights (4 B) and shadows (2 B), once
        # each with multicast stores, W-1 times with peer stores; in again: everybody else's shards
        wire_in = 4.0 * n * (world - 1) / world + 6.0 * shard * (world - 1)
        res["zero_floor_ms"] = wire_in / link * 1e3
        res["zero_fraction_of_link"] = res["zero_floor_ms"] / res["zero_fused_ms"]
        res["status"] = ctx.status()
        if rank == 0:
            print(json.dumps(res), flush=True)
    # vocab-parallel cross-entropy statistics of 2048 token rows: one kernel that exchanges (lse, target
    # logit) pairs and merges them, against three all-reduces (max, sum of exponentials, target logit)
    rows, shard = 2048, 16032
    merge = symm.VocabCEMerge(ctx)
    lse_l = torch.randn(rows, device=dev) + 10.0
    # local target index: inside [0, shard) on the rank that owns the row's target, outside elsewhere
    own = (torch.arange(rows, device=dev) % world) == rank
    t_l = torch.where(own, torch.randint(0, shard, (rows,), device=dev), torch.full((rows,), -1, device=dev))
    picked = torch.randn(rows, device=dev)
    row_loss = torch.where(own, lse_l - picked, torch.zeros_like(lse_l))
    res = {"case": "collectives", "world": world, "op": "vocab_ce_merge", "rows": rows}
    res["fused_ms"] = timed(lambda: merge(lse_l, row_loss, t_l, shard))

    def nccl_merge():   # the formulation the framework falls back to: one all-gather of (lse, target logit) pairs
        tgt = torch.where(own, lse_l - row_loss, torch.zeros_like(lse_l))
        stats = torch.stack([lse_l, tgt], dim=0).contiguous()
        allst = torch.empty((world,) + tuple(stats.shape), device=dev)
        dist.all_gather_into_tensor(allst.view(-1), stats.view(-1))
        return torch.logsumexp(allst[:, 0], dim=0) - allst[:, 1].sum(0)

    def nccl_three():   # the reference's three all-reduces: max, sum of exponentials, target logit
        m = lse_l.clone()
        dist.all_reduce(m, op=dist.ReduceOp.MAX)
        se = torch.exp(lse_l - m)
        dist.all_reduce(se)
        tl = torch.where(own, lse_l - row_loss, torch.zeros_like(lse_l))
        dist.all_reduce(tl)
        return m + torch.log(se) - tl

    res["nccl_allgather_ms"] = timed(nccl_merge)
    res["nccl_three_allreduces_ms"] = timed(nccl_three)
    # 8 bytes per row to every peer: latency-bound (two flag barriers), not bandwidth-bound
    res["floor_ms"] = 8.0 * rows * (world - 1) / link * 1e3
    res["status"] = ctx.status()
    if rank == 0:
        print(json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main(argv):
    C = _ext.load(required=True)
    torch.manual_seed(0)
    case = argv[1] if len(argv) > 1 else "gemm"
    {"gemm": bench_gemm, "gemm_llama_tp8": bench_gemm_llama_tp8, "gemm_probe": bench_gemm_probe, "norm": bench_norm, "attention": bench_attention, "profile": profile_case,
     "tp": bench_tp, "collectives": bench_collectives}[case](C)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
