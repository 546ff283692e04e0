"""LoRA behaviour (the assertions of the reference's tests/lora/test_lora.cc restated)."""
import math
import os

import pytest
import torch

from infinitrain_b200 import nn
from infinitrain_b200.nn import lora
from infinitrain_b200.nn.lora import LoRAConfig


@pytest.fixture(autouse=True)
def _env():
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    genv.InitAllEnv(world_size=1, rank=0)
    ProcessGroupFactory.Reset()
    ProcessGroupFactory.Instance().Init()


def test_config_scaling_and_matching():
    c = LoRAConfig(rank=4, alpha=8.0, target_modules={"c_attn", "attn.c_proj"})
    assert c.Scaling() == 2.0
    assert c.ShouldApplyLoRA("transformer.h.0.attn.c_attn")
    assert c.ShouldApplyLoRA("transformer.h.0.attn.c_proj")
    assert not c.ShouldApplyLoRA("transformer.h.0.mlp.c_proj")
    assert not c.ShouldApplyLoRA("transformer.h.0.mlp.c_fc")
    assert lora.ParseLoRATargetModules(" c_attn , attn.c_proj ,, ") == {"c_attn", "attn.c_proj"}


def test_lora_linear_shapes_and_freezing():
    c = LoRAConfig(rank=4, alpha=8.0)
    l = lora.LoRALinear(16, 8, c)
    assert tuple(l.lora_A.shape) == (4, 16) and tuple(l.lora_B.shape) == (8, 4)
    assert not l.weight.requires_grad and not l.bias.requires_grad
    assert l.lora_A.requires_grad and l.lora_B.requires_grad
    assert torch.count_nonzero(l.lora_B) == 0
    assert set(l.StateDict().keys()) == {"weight", "bias", "lora_A", "lora_B"}
    assert lora.CountTrainableParameters(l) == 4 * 16 + 8 * 4
    assert lora.CountTotalParameters(l) == 16 * 8 + 8 + 4 * 16 + 8 * 4


def test_merge_unmerge_roundtrip():
    torch.manual_seed(0)
    l = lora.LoRALinear(16, 8, LoRAConfig(rank=4, alpha=8.0))
    with torch.no_grad():
        l.lora_B.normal_()
    x = torch.randn(5, 16)
    w0 = l.weight.detach().clone()
    y0 = l(x)
    l.MergeWeights()
    assert l.IsMerged() and not l.lora_A.requires_grad and not l.lora_B.requires_grad
    assert abs((l(x) - y0).sum().item()) <= 1e-3
    l.UnmergeWeights()
    assert not l.IsMerged() and l.lora_A.requires_grad
    assert torch.allclose(l.weight, w0, atol=1e-6)
    l.MergeWeights()
    l.lora_A.requires_grad_(True)
    with pytest.raises(RuntimeError):
        l(x)


def test_inject_freeze_merge_and_unload_on_transformer(tmp_path):
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel

    torch.manual_seed(0)
    cfg = TransformerConfig.GPT2(n_layer=2, n_embd=32, n_head=2, n_kv_head=2, vocab_size=64, original_vocab_size=64,
                                 block_size=16)
    m = TransformerModel(cfg)
    total0 = lora.CountTotalParameters(m)
    m = lora.GetLoRAModel(m, LoRAConfig(rank=4, alpha=8.0, target_modules={"c_attn", "attn.c_proj"}))
    mods = [n for n, mod in m.NamedModules() if isinstance(mod, (lora.LoRAColumnParallelLinear, lora.LoRARowParallelLinear))]
    assert len(mods) == 4            # 2 layers x (c_attn, attn.c_proj); shared pipeline aliases listed once
    assert all("mlp" not in n for n in mods)
    tr = lora.CountTrainableParameters(m)
    assert tr == 2 * ((4 * 32 + 96 * 4) + (4 * 32 + 32 * 4))
    assert lora.CountTotalParameters(m) == total0 + tr
    assert len(lora.GetLoRAParameters(m)) == 8 and all(not p.requires_grad for p in lora.GetBaseParameters(m))
    idx = torch.randint(0, 64, (2, 16))
    with torch.no_grad():
        for p in lora.GetLoRAParameters(m):
            p.normal_(0, 0.05)
    y = m(idx)
    # adapter file round trip
    path = os.path.join(tmp_path, "adapter.bin")
    lora.SaveLoRAWeights(m, path)
    keep = {k: v.detach().clone() for k, v in lora.LoRAStateDict(m).items()}
    with torch.no_grad():
        for p in lora.GetLoRAParameters(m):
            p.zero_()
    lora.LoadLoRAWeights(m, path)
    for k, v in lora.LoRAStateDict(m).items():
        assert torch.equal(v, keep[k])
    with open(path, "rb") as f:
        assert int.from_bytes(f.read(4), "little") == 0x4C4F5241
    # training only moves the adapters
    from infinitrain_b200.optim import SGD

    base0 = [p.detach().clone() for p in lora.GetBaseParameters(m)]
    opt = SGD([p for p in m.parameters() if p.requires_grad], 0.1)
    nn.CrossEntropyLoss()(m(idx), idx).backward()
    opt.Step()
    assert all(torch.equal(a, b) for a, b in zip(base0, lora.GetBaseParameters(m)))
    y = m(idx)
    merged = lora.MergeAndUnload(m)
    assert not lora.LoRAStateDict(merged) and all(p.requires_grad for p in merged.parameters())
    assert lora.CountTotalParameters(merged) == total0
    assert torch.allclose(merged(idx), y, atol=1e-4)


def test_root_linear_matches_by_type_name():
    l = nn.Linear(8, 8)
    out = lora.InjectLoRALayers(l, LoRAConfig(rank=2, alpha=4, target_modules={"Linear"}))
    assert isinstance(out, lora.LoRALinear)
