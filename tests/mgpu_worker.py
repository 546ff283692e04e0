"""Worker of the multi-GPU tests; launched with torchrun, one process per GPU."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def setup():
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    genv.InitAllEnv(world_size=world, rank=rank)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    return rank, world, dev


def collectives():
    import torch.distributed as dist

    from infinitrain_b200.parallel import symm
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    rank, world, dev = setup()
    pg = ProcessGroupFactory.Instance().dp_group()
    ctx = symm.NvlinkContext.get(pg, dev)
    n = 1 << 20
    buf = ctx.alloc(n + 1024, torch.float32, dev)
    torch.manual_seed(rank)
    for it in range(3):
        buf[:n].normal_()
        ref = buf[:n].clone()
        dist.all_reduce(ref, op=dist.ReduceOp.AVG)
        ar = symm.BucketAllReduce(ctx, buf)
        w = ar(buf[256:n])   # a slice, as DDP buckets are
        assert w is not None
        w.WaitNonBlocking()
        torch.cuda.synchronize()
        err = (buf[256:n] - ref[256:]).abs().max().item()
        assert err < 1e-5, err
    assert ctx.status() == 0
    # fused reduce-scatter + AdamW + broadcast against NCCL + the single-GPU AdamW kernel
    C = ctx.C
    nb = 8 * world * 1000
    grads = ctx.alloc(nb, torch.float32, dev)
    params = ctx.alloc(nb, torch.float32, dev)
    shadow = ctx.alloc(nb, torch.bfloat16, dev)
    torch.manual_seed(100)
    init = torch.randn(nb, device=dev)
    params.copy_(init)
    torch.manual_seed(rank + 1)
    grads.normal_()
    gref = grads.clone()
    dist.all_reduce(gref, op=dist.ReduceOp.AVG)
    pref = init.clone()
    mref, vref = torch.zeros(nb, device=dev), torch.zeros(nb, device=dev)
    C.adamw(pref, gref, mref, vref, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0, None)

    class _B:  # minimal stand-ins for ParamAndGradBuffer / bucket
        grad_buffer, param_buffer, shadow_buffer = grads, params, shadow

    class _K:
        offset, numel = 0, nb

    m = torch.zeros(nb // world, device=dev)
    v = torch.zeros(nb // world, device=dev)
    step = symm.FusedZeroBucketStep(ctx, _B, _K, m, v)
    step(1e-2, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0 / world).WaitNonBlocking()
    torch.cuda.synchronize()
    dist.barrier()
    assert torch.allclose(params, pref, atol=1e-6, rtol=1e-5), (params - pref).abs().max().item()
    assert torch.equal(shadow, pref.bfloat16()) or (shadow.float() - pref).abs().max().item() < 1e-2
    assert ctx.status() == 0
    if rank == 0:
        print("COLLECTIVES OK multimem=%d" % int(ctx.ptrs(buf)[1] != 0))


def ddp(mode):
    import torch.distributed as dist

    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.models import GPT2
    from infinitrain_b200.nn import CrossEntropyLoss, init
    from infinitrain_b200.optim import Adam
    from infinitrain_b200.parallel.ddp.config import DistributedDataParallelConfig
    from infinitrain_b200.parallel.ddp.distributed_data_parallel import DistributedDataParallel
    from infinitrain_b200.parallel.ddp.distributed_optimizer import DistributedOptimizer

    rank, world, dev = setup()
    zero = int(mode[4])
    fused = not mode.endswith("nccl")

    def make():
        torch.manual_seed(0)
        init.manual_seed(42)
        return GPT2("gpt2", n_layer=2, block_size=128).to(dev)

    B, T, steps = 4, 128, 4
    g = torch.Generator().manual_seed(5)
    x = torch.randint(0, 50257, (B * world, T), generator=g).to(dev)
    y = torch.randint(0, 50257, (B * world, T), generator=g).to(dev)
    loss_fn = CrossEntropyLoss()

    def run(model, opt, xs, ys, ddp_mod=None):
        out = []
        for _ in range(steps):
            opt.ZeroGrad()
            with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16):
                loss = loss_fn(model(xs), ys)
            loss.backward()
            if ddp_mod is not None:
                ddp_mod.FinishGradSync()
            opt.Step()
            out.append(loss.detach().clone())
        return torch.stack(out)

    # oracle: single GPU, whole batch.  A large eps makes Adam's update nearly linear in the gradient, so
    # a gradient that arrives summed instead of averaged over the ranks (or scaled in any other way)
    # shows up in the update, which Adam's scale-invariant m / sqrt(v) would otherwise hide.
    kEps = 1e-3
    ref_model = make()
    init_params = [p.detach().clone() for p in ref_model.Parameters()]
    ref_opt = Adam(ref_model.Parameters(), 1e-3, eps=kEps)
    ref_losses = run(ref_model, ref_opt, x, y)
    ref_params = [p.detach().clone() for p in ref_model.Parameters()]

    model = make()
    cfg = DistributedDataParallelConfig(zero_stage=zero, use_fused_nvlink_kernels=fused)
    ddp_mod = DistributedDataParallel(model, config=cfg)
    creator = Adam.Create(1e-3, eps=kEps)
    opt = DistributedOptimizer(creator, ddp_mod.Parameters(), ddp_mod) if zero >= 1 else creator(ddp_mod.Parameters())
    if fused:
        assert ddp_mod.nvlink_ctx is not None, "fused NVLink kernels expected"
    losses = run(ddp_mod, opt, x.chunk(world)[rank], y.chunk(world)[rank], ddp_mod)
    dist.all_reduce(losses, op=dist.ReduceOp.AVG)
    assert (losses - ref_losses).abs().max().item() < 2e-2, (losses, ref_losses)
    worst, worst_at = 0.0, ""
    num = den = 0.0
    names = [n for n, _ in ddp_mod.named_parameters()]
    for k, (p, r, p0) in enumerate(zip(ddp_mod.Parameters(), ref_params, init_params)):
        rel = ((p - r).norm() / (r.norm() + 1e-9)).item()
        if rel > worst:
            worst, worst_at = rel, f"{names[k] if k < len(names) else k} {tuple(p.shape)}"
        num += float(((p - p0) - (r - p0)).double().pow(2).sum())
        den += float((r - p0).double().pow(2).sum())
    update_err = (num / max(den, 1e-30)) ** 0.5
    assert worst < 0.05, (worst, worst_at)
    # the four steps' total update, against the single-GPU run's: bf16 noise is a few per cent, a wrong
    # gradient scale is of order one
    assert update_err < 0.2, update_err
    if zero >= 1:
        # optimizer state of this rank's shards is on the averaged gradient's scale
        # (first and second moments of the shards, summed over the ranks, against the single-GPU run's)
        for name, mine, ref in (("m", opt.base_optimizer.m, ref_opt.m), ("v", opt.base_optimizer.v, ref_opt.v)):
            t = torch.tensor([sum(float(a.double().pow(2).sum()) for a in mine)], device=dev, dtype=torch.float64)
            dist.all_reduce(t)
            want = sum(float(a.double().pow(2).sum()) for a in ref)
            ratio = (t.item() / max(want, 1e-300)) ** 0.5
            assert 0.9 < ratio < 1.1, (name, ratio)
    if ddp_mod.nvlink_ctx is not None:
        assert ddp_mod.nvlink_ctx.status() == 0
    if rank == 0:
        print(f"DDP OK mode={mode} worst_rel={worst:.2e} update_err={update_err:.2e} losses={losses.tolist()}")


def tp_fused():
    """Column- and row-parallel linears under sequence parallelism: the fused all-gather+GEMM /
    GEMM+reduce-scatter launches against the NCCL formulation of the same layers."""
    import torch.distributed as dist

    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel import symm
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory
    from infinitrain_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    genv.InitAllEnv(world_size=world, rank=rank, tensor_parallel_size=world, sequence_parallel_enabled=True)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    B, Tl, H, F = 2, 256, 512, 1024 * world
    T = Tl * world
    torch.manual_seed(7)
    col = ColumnParallelLinear(H, F, bias=True, gather_output=False, input_is_parallel=False,
                               sequence_parallel=True, device=dev)
    col2 = ColumnParallelLinear(H, F, bias=False, gather_output=False, input_is_parallel=False,
                                sequence_parallel=True, device=dev)
    row = RowParallelLinear(F, H, bias=True, input_is_parallel=True, sequence_parallel=True, device=dev)
    torch.manual_seed(100 + rank)
    params = list(col.Parameters()) + list(col2.Parameters()) + list(row.Parameters())
    for prm in params:
        prm.data.normal_(0, 0.05)
    results = {}
    for fused in ("0", "1"):
        os.environ["ITB_FUSED_TP"] = fused
        symm.reset_fused_tp()
        outs = []
        for it in range(3):
            torch.manual_seed(1000 + it * 10 + rank)
            x = (torch.randn(B, Tl, H, device=dev) * 0.5).bfloat16().requires_grad_(True)
            res = (torch.randn(B, Tl, H, device=dev) * 0.5).bfloat16().requires_grad_(True)
            for prm in params:
                prm.grad = None
            with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16):
                # two column-parallel linears on one activation (the second reads the copy the first
                # gathered), as the gate / up projections of a SwiGLU MLP do
                h = col(x, gelu=(it % 2 == 1)) + col2(x)
                y = row(h, residual=res)
            assert y.shape == (B, Tl, H), y.shape
            torch.manual_seed(5000 + it * 10 + rank)
            gy = (torch.randn_like(y.float()) * 0.1).to(y.dtype)
            y.backward(gy)
            outs.append([y.detach().float(), x.grad.float(), res.grad.float()] +
                        [prm.grad.float().clone() for prm in params])
        torch.cuda.synchronize()
        results[fused] = outs
        if fused == "1":
            assert symm._TP_CTX is not None, "fused tensor-parallel context was not created"
            assert symm._TP_CTX.nvl.status() == 0, symm._TP_CTX.nvl.status()
            assert symm._TP_CTX.launch_index == 18, symm._TP_CTX.launch_index
    worst = 0.0
    names = ["y", "dx", "dres", "col.dw", "col.db", "col2.dw", "row.dw", "row.db"]
    for it, (a_it, b_it) in enumerate(zip(results["0"], results["1"])):
        for name, a, b in zip(names, a_it, b_it):
            rel = ((a - b).norm() / (a.norm() + 1e-6)).item()
            if rel > 2e-2:
                print(f"[rank {rank}] iteration {it} {name}: rel {rel:.3e}", flush=True)
            worst = max(worst, rel)
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() < 2e-2, t.item()
    if rank == 0:
        print(f"TP FUSED OK worst_rel={t.item():.2e}")


def tp_fused_nosp():
    """Tensor parallelism without sequence parallelism: the GEMM + all-reduce launches (row-parallel
    forward, column-parallel backward) against the NCCL formulation."""
    import torch.distributed as dist

    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel import symm
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory
    from infinitrain_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    genv.InitAllEnv(world_size=world, rank=rank, tensor_parallel_size=world, sequence_parallel_enabled=False)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    B, T, H, F = 2, 256 * world, 512, 1024 * world
    col = ColumnParallelLinear(H, F, bias=True, gather_output=False, input_is_parallel=False, device=dev)
    row = RowParallelLinear(F, H, bias=True, input_is_parallel=True, device=dev)
    torch.manual_seed(100 + rank)
    params = list(col.Parameters()) + list(row.Parameters())
    for prm in params:
        prm.data.normal_(0, 0.05)
    dist.broadcast(row.bias.data, 0)           # a replicated parameter
    results = {}
    for fused in ("0", "1"):
        os.environ["ITB_FUSED_TP"] = fused
        symm.reset_fused_tp()
        outs = []
        for it in range(3):
            torch.manual_seed(1000 + it)       # activations are replicated: same on every rank
            x = (torch.randn(B, T, H, device=dev) * 0.5).bfloat16().requires_grad_(True)
            res = (torch.randn(B, T, H, device=dev) * 0.5).bfloat16().requires_grad_(True)
            gy = (torch.randn(B, T, H, device=dev) * 0.1).bfloat16()
            for prm in params:
                prm.grad = None
            with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16):
                y = row(col(x, gelu=(it % 2 == 1)), residual=res)
            assert y.shape == (B, T, H)
            y.backward(gy)
            outs.append([y.detach().float(), x.grad.float(), res.grad.float()] + [p.grad.float().clone() for p in params])
        torch.cuda.synchronize()
        results[fused] = outs
        if fused == "1":
            assert symm._TP_CTX is not None and symm._TP_CTX.nvl.status() == 0
            assert symm._TP_CTX.launch_index == 6, symm._TP_CTX.launch_index
    worst = 0.0
    names = ["y", "dx", "dres", "col.dw", "col.db", "row.dw", "row.db"]
    for it, (a_it, b_it) in enumerate(zip(results["0"], results["1"])):
        for name, a, b in zip(names, a_it, b_it):
            rel = ((a - b).norm() / (a.norm() + 1e-6)).item()
            if rel > 2e-2:
                print(f"[rank {rank}] iteration {it} {name}: rel {rel:.3e}", flush=True)
            worst = max(worst, rel)
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() < 2e-2, t.item()
    if rank == 0:
        print(f"TP NOSP OK worst_rel={t.item():.2e}")


def tp_model():
    """A small LLaMA-3-shaped model under TP + SP trained for a few steps: the loss trajectory with the
    fused all-gather+GEMM / GEMM+reduce-scatter / CE-merge kernels against the NCCL formulation of the
    same model from the same weights."""
    import torch.distributed as dist

    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.models import LLaMA3
    from infinitrain_b200.nn import init
    from infinitrain_b200.optim import Adam
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel import symm
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory
    from infinitrain_b200.parallel.tensor_parallel import AllReduceSequenceParallelGrads, VocabParallelCrossEntropyLoss

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    genv.InitAllEnv(world_size=world, rank=rank, tensor_parallel_size=world, sequence_parallel_enabled=True)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    B, T, V, steps = 2, 256 * world, 2048, 4
    g = torch.Generator().manual_seed(5)
    x = torch.randint(0, V, (B, T), generator=g).to(dev)
    y = torch.randint(0, V, (B, T), generator=g).to(dev)
    curves = {}
    for fused in ("0", "1"):
        os.environ["ITB_FUSED_TP"] = fused
        symm.reset_fused_tp()
        torch.manual_seed(0)
        init.manual_seed(42 + rank)
        model = LLaMA3("llama3-1b", n_layer=2, n_embd=512, n_head=8, n_kv_head=4, vocab_size=V, original_vocab_size=V,
                       block_size=T).to(dev)
        loss_fn = VocabParallelCrossEntropyLoss(V)
        opt = Adam(model.Parameters(), 1e-3)
        out = []
        for _ in range(steps):
            opt.ZeroGrad()
            with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16):
                loss = loss_fn(model(x), y)
            loss.backward()
            AllReduceSequenceParallelGrads(model)
            opt.Step()
            out.append(loss.detach().float().clone())
        torch.cuda.synchronize()
        curves[fused] = torch.stack(out)
        if fused == "1":
            assert symm._TP_CTX is not None and symm._TP_CTX.nvl.status() == 0
            assert symm._TP_CTX.launch_index > 0
    a, b = curves["0"], curves["1"]
    assert a[-1] < a[0] and b[-1] < b[0], (a.tolist(), b.tolist())
    assert (a - b).abs().max().item() < 5e-2, (a.tolist(), b.tolist())
    if rank == 0:
        print(f"TP MODEL OK nccl={[round(v, 4) for v in a.tolist()]} fused={[round(v, 4) for v in b.tolist()]}")


def pp_gpu():
    """Two pipeline stages on two GPUs, bf16 autocast, virtual stages: the interleaved 1F1B and the
    GPipe order of the same micro-batches give the same loss trajectory, and it decreases."""
    import hashlib
    import re

    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.nn import CrossEntropyLoss
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.optim import SGD
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.pp.pipeline_parallel import PipelineParallel
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    vpp = 2
    genv.InitAllEnv(world_size=world, rank=rank, pipeline_parallel_size=world, virtual_pipeline_parallel=vpp)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    cfg = TransformerConfig.LLaMA3(n_layer=4, n_embd=256, n_head=4, n_kv_head=2, vocab_size=512, original_vocab_size=512,
                                   block_size=128, multiple_of=64)
    B, T, n_mb, steps = 8, 128, 4, 3
    g = torch.Generator().manual_seed(1)
    x = torch.randint(0, 512, (B, T), generator=g).to(dev)
    y = torch.randint(0, 512, (B, T), generator=g).to(dev)
    curves = {}
    for schedule in ("1f1b", "gpipe"):
        model = TransformerModel(cfg).to(dev)
        offs = [l for (s0, e0) in sorted(model.stage_info.layer_ranges_per_chunk) for l in range(s0, e0)]
        with torch.no_grad():
            for name, p in model.StateDict().items():
                m = re.match(r"transformer\.h\.(\d+)\.(.*)", name)
                gname = f"transformer.h.{offs[int(m.group(1))]}.{m.group(2)}" if m else name
                gen = torch.Generator().manual_seed(int(hashlib.md5(gname.encode()).hexdigest()[:8], 16))
                p.copy_((torch.randn(p.shape, generator=gen) * 0.05 + (1.0 if p.dim() == 1 else 0.0)).to(dev))
        pp = PipelineParallel(model, world, n_mb, [B // n_mb, T, cfg.n_embd], rank, dev, vpp, schedule=schedule)
        opt = SGD(pp.Parameters(), 0.05)
        out = []
        for _ in range(steps):
            out.append(float(pp.TrainStep([x], [y], opt, CrossEntropyLoss(), DataType.kBFLOAT16)))
        torch.cuda.synchronize()
        curves[schedule] = out
    if rank == world - 1:
        a, b = curves["1f1b"], curves["gpipe"]
        assert all(v == v for v in a) and a[-1] < a[0], a
        assert max(abs(u - v) for u, v in zip(a, b)) < 2e-2, (a, b)
        print(f"PP GPU OK 1f1b={[round(v, 4) for v in a]} gpipe={[round(v, 4) for v in b]}")


def vocab_ce():
    """Vocab-parallel cross-entropy: the NVLink merge kernel against the all-gather formulation and
    against the loss over the gathered full-vocabulary logits."""
    import torch.distributed as dist

    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel import symm
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory
    from infinitrain_b200.parallel.tensor_parallel import VocabParallelCrossEntropyLoss

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    genv.InitAllEnv(world_size=world, rank=rank, tensor_parallel_size=world, sequence_parallel_enabled=True)
    ProcessGroupFactory.Instance().Init(device=dev, timeout_s=120)
    B, T, V_local = 2, 600, 1000
    V_orig = V_local * world - 37            # the last shard is partly padding
    loss_fn = VocabParallelCrossEntropyLoss(V_orig)
    outs = {}
    for fused in ("0", "1"):
        os.environ["ITB_FUSED_TP"] = fused
        symm.reset_fused_tp()
        res = []
        for it in range(3):
            torch.manual_seed(77 + it)                      # same targets on every rank
            target = torch.randint(0, V_orig, (B, T), device=dev)
            torch.manual_seed(1000 * it + rank)
            logits = (torch.randn(B, T, V_local, device=dev) * 2).bfloat16().requires_grad_(True)
            keep = logits.detach().clone()      # the backward pass writes the gradient over the logits
            loss = loss_fn(logits, target)
            loss.backward()
            res.append((loss.detach().float().clone(), logits.grad.float().clone(), keep, target))
        torch.cuda.synchronize()
        outs[fused] = res
        if fused == "1":
            assert symm._TP_CTX is not None and symm._TP_CTX.nvl.status() == 0
    for (l0, g0, lg, tg), (l1, g1, _, _) in zip(outs["0"], outs["1"]):
        assert abs(l0.item() - l1.item()) < 1e-4 * max(1.0, abs(l0.item())), ("nccl vs fused", l0.item(), l1.item())
        assert ((g0 - g1).norm() / (g0.norm() + 1e-9)).item() < 1e-3, "gradients differ"
        # full-vocabulary reference from the gathered shards
        full = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(full, lg.contiguous())
        ref = torch.nn.functional.cross_entropy(torch.cat(full, -1)[..., :V_orig].float().view(B * T, -1), tg.view(-1))
        assert abs(ref.item() - l1.item()) < 2e-3 * max(1.0, abs(ref.item())), ("full vocab vs fused", ref.item(), l1.item())
    if rank == 0:
        print("VOCAB CE OK")


if __name__ == "__main__":
    if sys.argv[1] == "vocab_ce":
        vocab_ce()
    elif sys.argv[1] == "tp_fused_nosp":
        tp_fused_nosp()
    elif sys.argv[1] == "tp_model":
        tp_model()
    elif sys.argv[1] == "pp_gpu":
        pp_gpu()
    elif sys.argv[1] == "collectives":
        collectives()
    elif sys.argv[1] == "tp_fused":
        tp_fused()
    else:
        ddp(sys.argv[2])
    import torch.distributed as dist

    dist.barrier()
    dist.destroy_process_group()
