"""llm.c weight files: write -> read round trip, tensor-parallel sharding rules."""
import os

import numpy as np
import pytest
import torch

from dist_utils import run_ranks
from infinitrain_b200.models import llmc
from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel


def _single_env():
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    genv.InitAllEnv(world_size=1, rank=0)
    ProcessGroupFactory.Reset()
    ProcessGroupFactory.Instance().Init()


def _gpt2_cfg():
    return TransformerConfig.GPT2(n_layer=2, n_embd=32, n_head=4, n_kv_head=4, vocab_size=100, original_vocab_size=100,
                                  block_size=16)


def _llama_cfg():
    return TransformerConfig.LLaMA3(n_layer=2, n_embd=32, n_head=4, n_kv_head=2, vocab_size=96, original_vocab_size=96,
                                    block_size=16, multiple_of=16, ffn_dim_multiplier=1.5)


@pytest.mark.parametrize("family", ["gpt2", "llama3"])
def test_roundtrip_single_rank(tmp_path, family):
    _single_env()
    torch.manual_seed(0)
    cfg = _gpt2_cfg() if family == "gpt2" else _llama_cfg()
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.02)
    path = os.path.join(tmp_path, "w.bin")
    if family == "gpt2":
        llmc.write_gpt2_llmc(path, cfg, llmc.full_state_dict(m))
        h = np.fromfile(path, dtype=np.int32, count=8)
        assert list(h) == [20240326, 3, 16, 100, 2, 4, 32, 128]
        m2 = llmc.GPT2FromLLMC(path)
    else:
        llmc.write_llama3_llmc(path, cfg, llmc.full_state_dict(m))
        m2 = llmc.LLaMA3FromLLMC(path)
        assert m2.config.ffn_hidden() == cfg.ffn_hidden() and m2.config.n_kv_head == 2
    a, b = m.StateDict(), m2.StateDict()
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k
    x = torch.randint(0, 90, (2, 16))
    assert torch.allclose(m(x), m2(x))


def _tp_worker(rank, world, path, full_logits):
    from infinitrain_b200.parallel import tensor_parallel as tpm

    m = llmc.LLaMA3FromLLMC(path)
    g = torch.Generator().manual_seed(3)
    x = torch.randint(0, 90, (2, 16), generator=g)
    local = m(x)                                   # [B, T, V / tp]
    gathered = tpm._gather_along(local, tpm._tp(), 2)
    assert torch.allclose(gathered, full_logits, atol=1e-5), (gathered - full_logits).abs().max()


@pytest.mark.parametrize("sp", [False, True])
def test_tp2_sharded_load_reproduces_full_model(tmp_path, sp):
    _single_env()
    torch.manual_seed(1)
    cfg = _llama_cfg()
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.05)
    path = os.path.join(tmp_path, "w.bin")
    llmc.write_llama3_llmc(path, cfg, llmc.full_state_dict(m))
    g = torch.Generator().manual_seed(3)
    x = torch.randint(0, 90, (2, 16), generator=g)
    run_ranks(_tp_worker, 2, args=(path, m(x).detach()), tp=2, sp=sp)
