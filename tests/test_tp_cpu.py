"""Tensor / sequence parallel training on CPU ranks (gloo) against the unpartitioned model."""
import os

import pytest
import torch

from dist_utils import run_ranks
from infinitrain_b200.models import llmc
from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel


def _cfg(family):
    if family == "gpt2":
        return TransformerConfig.GPT2(n_layer=2, n_embd=32, n_head=4, n_kv_head=4, vocab_size=96, original_vocab_size=90,
                                      block_size=16)
    return TransformerConfig.LLaMA3(n_layer=2, n_embd=32, n_head=4, n_kv_head=2, vocab_size=96, original_vocab_size=90,
                                    block_size=16, multiple_of=16)


def _data():
    g = torch.Generator().manual_seed(3)
    return torch.randint(0, 90, (2, 16), generator=g), torch.randint(0, 90, (2, 16), generator=g)


def _tp_train_worker(rank, world, family, path, ref_losses):
    from infinitrain_b200.optim import SGD
    from infinitrain_b200.parallel.tensor_parallel import AllReduceSequenceParallelGrads, VocabParallelCrossEntropyLoss

    m = llmc.GPT2FromLLMC(path) if family == "gpt2" else llmc.LLaMA3FromLLMC(path)
    opt = SGD(m.Parameters(), 0.05)
    loss_fn = VocabParallelCrossEntropyLoss(90)
    x, y = _data()
    for s in range(3):
        opt.ZeroGrad()
        loss = loss_fn(m(x), y)
        loss.backward()
        AllReduceSequenceParallelGrads(m)
        opt.Step()
        assert abs(loss.item() - ref_losses[s]) < 2e-5, (s, loss.item(), ref_losses[s])


@pytest.mark.parametrize("family,sp", [("llama3", False), ("llama3", True), ("gpt2", True)])
def test_tp2_training_matches_unpartitioned(tmp_path, family, sp):
    from infinitrain_b200.optim import SGD
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory
    from infinitrain_b200.parallel.tensor_parallel import VocabParallelCrossEntropyLoss

    genv.InitAllEnv(world_size=1, rank=0)
    ProcessGroupFactory.Reset()
    ProcessGroupFactory.Instance().Init()
    torch.manual_seed(2)
    cfg = _cfg(family)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.05)
        # padded vocabulary rows (>= original vocab) are zero in llm.c files
        m.lm_head.weight[90:].zero_()
    path = os.path.join(tmp_path, "w.bin")
    if family == "gpt2":
        llmc.write_gpt2_llmc(path, cfg, llmc.full_state_dict(m), padded_vocab_size=96)
    else:
        llmc.write_llama3_llmc(path, cfg, llmc.full_state_dict(m))
    opt = SGD(m.Parameters(), 0.05)
    loss_fn = VocabParallelCrossEntropyLoss(90)
    x, y = _data()
    ref = []
    for _ in range(3):
        opt.ZeroGrad()
        loss = loss_fn(m(x), y)
        loss.backward()
        opt.Step()
        ref.append(loss.item())
    run_ranks(_tp_train_worker, 2, args=(family, path, ref), tp=2, sp=sp)
