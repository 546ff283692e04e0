"""Architecture facts of the Transformer building blocks on CPU: parameter counts, output shapes,
RoPE table shape, state-dict coverage (the assertions of the reference's
tests/transformer/test_transformer_architecture.cc:59-190)."""
import pytest
import torch

from infinitrain_b200 import nn
from infinitrain_b200.models.gpt2 import GPT2
from infinitrain_b200.models.llama3 import llama3_config
from infinitrain_b200.nn.transformer.config import AttentionType, MLPType, NormType, TransformerConfig
from infinitrain_b200.nn.transformer.modules import (MLP, CausalSelfAttention, PrecomputeFreqsCis, TransformerLayer)
from infinitrain_b200.parallel import global_env as genv


@pytest.fixture(autouse=True)
def single_rank_env():
    genv.InitAllEnv(world_size=1, rank=0)
    yield


def _gpt_cfg(**kw):
    return TransformerConfig(block_size=32, vocab_size=128, original_vocab_size=128, n_layer=2, n_head=4, n_kv_head=4,
                             n_embd=32, **kw)


def _llama_cfg(**kw):
    return TransformerConfig(block_size=32, vocab_size=128, original_vocab_size=128, n_layer=2, n_head=4, n_kv_head=2,
                             n_embd=32, attention_type=AttentionType.kRoPE, activation_type=MLPType.kSwiGLU,
                             norm_type=NormType.kRMSNorm, add_bias_linear=False, tie_weights=False, multiple_of=16, **kw)


def test_basic_layers_shapes_and_parameter_counts():
    emb = nn.Embedding(100, 16)
    assert emb(torch.randint(0, 100, (2, 5))).shape == (2, 5, 16) and len(list(emb.Parameters())) == 1
    ln = nn.LayerNorm(16)
    assert ln(torch.randn(2, 5, 16)).shape == (2, 5, 16) and len(list(ln.Parameters())) == 2
    rn = nn.RMSNorm(16)
    assert rn(torch.randn(2, 5, 16)).shape == (2, 5, 16) and len(list(rn.Parameters())) == 1
    lin = nn.Linear(16, 8)
    assert lin.weight.shape == (8, 16) and lin.bias.shape == (8,)


def test_mlp_and_attention_parameter_counts():
    assert len(list(MLP(_gpt_cfg()).Parameters())) == 4              # c_fc w/b, c_proj w/b
    assert len(list(MLP(_llama_cfg()).Parameters())) == 3            # c_fc, c_fc2, c_proj, no biases
    assert len(list(CausalSelfAttention(_gpt_cfg()).Parameters())) == 4
    assert len(list(CausalSelfAttention(_llama_cfg()).Parameters())) == 2
    a = CausalSelfAttention(_llama_cfg())
    assert a.c_attn.weight.shape == ((4 + 2 * 2) * 8, 32) and a.n_rep == 2


def test_ffn_width_rule():
    # GELU: 4x; SwiGLU: 2/3 of 4x, times the multiplier, rounded up to multiple_of
    assert _gpt_cfg(ffn_dim_multiplier=None).ffn_hidden() % 256 == 0
    c = _llama_cfg(ffn_dim_multiplier=1.5)
    h = int(2 * (32 * 4)) // 3
    assert c.ffn_hidden() == -(-int(round(h * 1.5)) // 16) * 16


def test_rope_table_shape_and_values():
    t = PrecomputeFreqsCis(64, 128)
    assert tuple(t.shape) == (128, 32, 2)
    assert torch.allclose(t[0, :, 0], torch.ones(32)) and torch.allclose(t[0, :, 1], torch.zeros(32))
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2).float() / 64))
    assert torch.allclose(t[5, :, 0], torch.cos(5 * inv), atol=1e-6)
    assert torch.allclose(t[5, :, 1], torch.sin(5 * inv), atol=1e-6)


@pytest.mark.parametrize("cfg", [_gpt_cfg, _llama_cfg])
def test_layer_and_model_shapes(cfg):
    from infinitrain_b200.nn.transformer.modules import TransformerModel

    c = cfg()
    layer = TransformerLayer(c)
    x = torch.randn(2, 8, 32)
    fc = PrecomputeFreqsCis(c.head_dim(), 64, c.rope_theta)[:8] if c.attention_type == AttentionType.kRoPE else None
    assert layer(x, fc, 0).shape == (2, 8, 32)
    m = TransformerModel(c)
    logits = m(torch.randint(0, 128, (2, 8)))
    assert logits.shape == (2, 8, 128)
    params = list(m.Parameters())
    sd = m.StateDict()
    assert len(sd) >= len(params)
    assert len({id(p) for p in params}) == len(params)              # Parameters() has no duplicates
    if c.tie_weights:
        assert sd["transformer.wte.weight"].data_ptr() == sd["lm_head.weight"].data_ptr()
        n_expected = 2 + 2 * 12 + 2                                   # wte(+head), wpe, 12 per layer, ln_f w/b
    else:
        n_expected = 1 + 2 * 5 + 1 + 1 + 2 * 2                        # wte, 5 linears/layer, ln_f, head, 2 norms/layer
    assert len(params) == n_expected
    logits.float().sum().backward()
    assert all(p.grad is not None or getattr(p, "main_grad", None) is not None for p in params)


def test_named_models_have_the_published_sizes():
    def count(m):
        return sum(p.numel() for p in m.Parameters())

    assert count(GPT2("gpt2")) == 124_439_808                        # the published 124M (vocabulary 50257)
    c = llama3_config("llama3-8b")
    assert (c.n_layer, c.n_embd, c.n_head, c.n_kv_head, c.head_dim(), c.ffn_hidden(), c.vocab_size) == \
        (32, 4096, 32, 8, 128, 14336, 128256)
    per_layer = 4096 * (32 + 16) * 128 + 4096 * 4096 + 3 * 4096 * 14336 + 2 * 4096
    assert 2 * 128256 * 4096 + 32 * per_layer + 4096 == 8_030_261_248   # the published 8.03 B


def test_state_dict_names_follow_the_reference_layout():
    from infinitrain_b200.nn.transformer.modules import TransformerModel

    sd = TransformerModel(_gpt_cfg()).StateDict()
    for k in ("transformer.wte.weight", "transformer.wpe.weight", "transformer.h.0.ln_1.weight",
              "transformer.h.0.attn.c_attn.weight", "transformer.h.0.attn.c_proj.bias", "transformer.h.1.mlp.c_fc.weight",
              "transformer.h.1.mlp.c_proj.weight", "transformer.ln_f.bias", "lm_head.weight"):
        assert k in sd, k
    assert not any(k.startswith("__pp") for k in sd)
