"""Pipeline parallelism: schedule invariants (pure) and 2-stage training on CPU ranks (gloo) against
single-process training with gradient accumulation over the same micro-batches."""
import pytest
import torch

from dist_utils import run_ranks
from infinitrain_b200.parallel.pp.schedule import (GenerateGPipeSchedule, GenerateInterleaved1F1BSchedule,
                                                   ValidateSchedule)
from infinitrain_b200.parallel.pp.stage_info import GetStageInfo


@pytest.mark.parametrize("n,S,V", [(4, 2, 1), (8, 2, 2), (8, 4, 2), (3, 4, 1), (1, 2, 2), (16, 8, 1)])
def test_schedules_are_valid(n, S, V):
    for gen in (GenerateGPipeSchedule, GenerateInterleaved1F1BSchedule):
        ValidateSchedule(gen(n, S, V), n, S, V)


def test_gpipe_matches_documented_steps():
    n, S, V = 3, 2, 1
    sch = GenerateGPipeSchedule(n, S, V)
    T = n + S * V - 1
    for t in sch:
        if t.is_forward:
            assert t.step == t.microbatch_id + t.global_chunk_id
        else:
            assert t.step == T + (T - 1 - t.global_chunk_id - t.microbatch_id)
    assert [t.step for t in sch] == sorted(t.step for t in sch)


def test_1f1b_bounds_in_flight_microbatches():
    n, S, V = 16, 4, 1
    for stage in range(S):
        live = peak = 0
        for t in GenerateInterleaved1F1BSchedule(n, S, V):
            if t.stage_id != stage:
                continue
            live += 1 if t.is_forward else -1
            peak = max(peak, live)
        assert peak <= 2 * S * V - 1, (stage, peak)  # bounded by the pipeline depth; GPipe holds all 16
    peak_gpipe = 0
    live = 0
    for t in GenerateGPipeSchedule(n, S, V):
        if t.stage_id == 0:
            live += 1 if t.is_forward else -1
            peak_gpipe = max(peak_gpipe, live)
    assert peak_gpipe == n


def test_stage_info_round_robin_with_remainder():
    assert GetStageInfo(16, 2, 0, 2).layer_ranges_per_chunk == [(0, 4), (8, 12)]
    assert GetStageInfo(16, 2, 1, 2).layer_ranges_per_chunk == [(4, 8), (12, 16)]
    # 14 layers over 4 chunks: the first two chunks get 4 layers, the others 3
    got = [GetStageInfo(14, 4, r, 1).layer_ranges_per_chunk for r in range(4)]
    assert got == [[(0, 4)], [(4, 8)], [(8, 11)], [(11, 14)]]
    assert GetStageInfo(12, 4, 0, 1).is_first_stage and GetStageInfo(12, 4, 3, 1).is_last_stage


def _cfg():
    from infinitrain_b200.nn.transformer import TransformerConfig

    return TransformerConfig.LLaMA3(n_layer=4, n_embd=32, n_head=4, n_kv_head=2, vocab_size=64, original_vocab_size=64,
                                    block_size=16, multiple_of=16)


def _full_state(seed=11):
    """Weights of the whole (unpartitioned) model, generated deterministically by name."""
    from infinitrain_b200.parallel import global_env as genv

    return seed


def _init_by_name(model, layer_offsets):
    """Deterministic init keyed by the GLOBAL parameter name so that partitioned and full models
    agree.  ``layer_offsets`` maps local layer index -> global layer index."""
    import hashlib
    import re

    with torch.no_grad():
        for name, p in model.StateDict().items():
            m = re.match(r"transformer\.h\.(\d+)\.(.*)", name)
            gname = f"transformer.h.{layer_offsets[int(m.group(1))]}.{m.group(2)}" if m else name
            seed = int(hashlib.md5(gname.encode()).hexdigest()[:8], 16)
            g = torch.Generator().manual_seed(seed)
            p.copy_(torch.randn(p.shape, generator=g) * 0.05 + (1.0 if p.dim() == 1 else 0.0))


def _pp_worker(rank, world, vpp, schedule, n_mb, ref_loss, ref_params):
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.nn import CrossEntropyLoss
    from infinitrain_b200.nn.transformer import TransformerModel
    from infinitrain_b200.optim import SGD
    from infinitrain_b200.parallel.pp.pipeline_parallel import PipelineParallel

    cfg = _cfg()
    model = TransformerModel(cfg)
    offs = [l for (s, e) in sorted(model.stage_info.layer_ranges_per_chunk) for l in range(s, e)]
    _init_by_name(model, offs)
    B, T = 8, 16
    g = torch.Generator().manual_seed(1)
    x = torch.randint(0, 64, (B, T), generator=g)
    y = torch.randint(0, 64, (B, T), generator=g)
    pp = PipelineParallel(model, world, n_mb, [B // n_mb, T, cfg.n_embd], rank, torch.device("cpu"), vpp,
                          schedule=schedule)
    opt = SGD(pp.Parameters(), 0.1)
    loss = pp.TrainStep([x], [y], opt, CrossEntropyLoss(), DataType.kFLOAT32)
    if rank == world - 1:
        assert abs(loss - ref_loss) < 1e-5, (loss, ref_loss)
    import re

    for name, p in model.StateDict().items():
        m = re.match(r"transformer\.h\.(\d+)\.(.*)", name)
        gname = f"transformer.h.{offs[int(m.group(1))]}.{m.group(2)}" if m else name
        assert torch.allclose(p, ref_params[gname], atol=1e-5), gname


@pytest.mark.parametrize("vpp,schedule", [(1, "1f1b"), (2, "1f1b"), (2, "gpipe")])
def test_two_stage_pipeline_matches_single_process(vpp, schedule):
    from infinitrain_b200.nn import CrossEntropyLoss
    from infinitrain_b200.nn.transformer import TransformerModel
    from infinitrain_b200.optim import SGD
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    genv.InitAllEnv(world_size=1, rank=0)
    ProcessGroupFactory.Reset()
    ProcessGroupFactory.Instance().Init()
    n_mb = 4
    model = TransformerModel(_cfg())
    _init_by_name(model, list(range(4)))
    g = torch.Generator().manual_seed(1)
    x = torch.randint(0, 64, (8, 16), generator=g)
    y = torch.randint(0, 64, (8, 16), generator=g)
    opt = SGD(model.Parameters(), 0.1)
    opt.ZeroGrad()
    total = 0.0
    for xm, ym in zip(x.chunk(n_mb), y.chunk(n_mb)):
        loss = CrossEntropyLoss()(model(xm), ym) / n_mb
        loss.backward()
        total += loss.item()
    opt.Step()
    ref_params = {k: v.detach().clone() for k, v in model.StateDict().items()}
    run_ranks(_pp_worker, 2, args=(vpp, schedule, n_mb, total, ref_params), pp=2, vpp=vpp)
