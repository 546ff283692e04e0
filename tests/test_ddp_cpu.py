"""Data parallelism on CPU ranks (gloo): every DDP mode must reproduce the single-process result
on the concatenated batch."""
import copy

import pytest
import torch

from dist_utils import run_ranks


def _tiny_model():
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel

    from infinitrain_b200.nn import init

    torch.manual_seed(7)
    init.manual_seed(42)
    cfg = TransformerConfig.GPT2(n_layer=2, n_embd=32, n_head=2, n_kv_head=2, vocab_size=97, original_vocab_size=97,
                                 block_size=16)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.05)
    return m


def _data(world, per_rank=2, T=16):
    g = torch.Generator().manual_seed(3)
    x = torch.randint(0, 97, (world * per_rank, T), generator=g)
    y = torch.randint(0, 97, (world * per_rank, T), generator=g)
    return x, y


def _reference_run(world, steps, lr=1e-2):
    """Single process, full batch, plain Adam: the oracle."""
    from infinitrain_b200.nn import CrossEntropyLoss
    from infinitrain_b200.optim import Adam

    m = _tiny_model()
    opt = Adam(m.Parameters(), lr)
    x, y = _data(world)
    losses = []
    for _ in range(steps):
        opt.ZeroGrad()
        loss = CrossEntropyLoss()(m(x), y)
        loss.backward()
        opt.Step()
        losses.append(loss.item())
    return losses, [p.detach().clone() for p in m.Parameters()]


def _ddp_worker(rank, world, zero_stage, bucketing, steps, ref_losses, ref_params):
    from infinitrain_b200.nn import CrossEntropyLoss
    from infinitrain_b200.optim import Adam
    from infinitrain_b200.parallel.ddp.config import DistributedDataParallelConfig
    from infinitrain_b200.parallel.ddp.distributed_data_parallel import DistributedDataParallel
    from infinitrain_b200.parallel.ddp.distributed_optimizer import DistributedOptimizer
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory, ReduceOpType

    m = _tiny_model()
    if rank != 0:  # DDP must broadcast rank 0's weights
        with torch.no_grad():
            for p in m.parameters():
                p.add_(1.0)
    cfg = DistributedDataParallelConfig(zero_stage=zero_stage, gradient_bucketing_enabled=bucketing,
                                        bucket_size_in_elements=2000, first_bucket_cap_mb=0, normal_bucket_cap_mb=0)
    ddp = DistributedDataParallel(m, config=cfg)
    creator = Adam.Create(1e-2)
    opt = DistributedOptimizer(creator, ddp.Parameters(), ddp) if zero_stage >= 1 else creator(ddp.Parameters())
    x, y = _data(world)
    xs, ys = x.chunk(world)[rank], y.chunk(world)[rank]
    pg = ProcessGroupFactory.Instance().dp_group()
    for s in range(steps):
        opt.ZeroGrad()
        loss = CrossEntropyLoss()(ddp(xs), ys)
        loss.backward()
        ddp.FinishGradSync()
        opt.Step()
        l = loss.detach().clone()
        pg.AllReduce(l, ReduceOpType.kAvg)
        assert abs(l.item() - ref_losses[s]) < 1e-4, (s, l.item(), ref_losses[s])
    for p, r in zip(ddp.Parameters(), ref_params):
        assert torch.allclose(p, r, atol=5e-4, rtol=1e-3), (p - r).abs().max()


@pytest.mark.parametrize("zero_stage,bucketing", [(0, True), (0, False), (1, True), (2, True)])
def test_ddp_matches_single_process(zero_stage, bucketing):
    world, steps = 2, 3
    ref_losses, ref_params = _reference_run(world, steps)
    run_ranks(_ddp_worker, world, args=(zero_stage, bucketing, steps, ref_losses, ref_params))


def test_ddp_zero2_four_ranks():
    world, steps = 4, 2
    ref_losses, ref_params = _reference_run(world, steps)
    run_ranks(_ddp_worker, world, args=(2, True, steps, ref_losses, ref_params))


def test_bucket_assignment_and_flat_layout():
    from infinitrain_b200.parallel.ddp.param_and_grad_buffer import plan_flat_layout
    from infinitrain_b200.parallel.ddp.reducer import ComputeBucketAssignmentBySize

    ts = [torch.zeros(n) for n in (10, 300000, 20, 400000, 5)]   # fp32: 4 bytes each
    b = ComputeBucketAssignmentBySize(ts, [1 << 20, 25 << 20])
    # reverse walk: 5, 400000 (1.6 MB >= 1 MB cap -> flush), then 20, 300000, 10 under the 25 MB cap
    assert b == [[4, 3], [2, 1, 0]]
    lay = plan_flat_layout([100, 1_000_000, 50], dp_size=8, shard=True)
    # reverse order; every start a multiple of 64; bucket closes at >= 1M elements; end padded to lcm(8,128)
    assert lay.param_ranges[2] == (0, 50, 0)
    assert lay.param_ranges[1] == (64, 1_000_064, 0)
    assert lay.bucket_ranges[0] == (0, 1_000_064)
    assert lay.param_ranges[0][0] == 1_000_064 and lay.param_ranges[0][2] == 1
    assert lay.bucket_ranges[1][1] % 128 == 0 and lay.numel % 8 == 0
    lay0 = plan_flat_layout([100, 1_000_000, 50], dp_size=8, shard=False)
    assert lay0.numel == lay0.numel_unpadded == 1_000_150
