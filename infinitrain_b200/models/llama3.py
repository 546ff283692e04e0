"""LLaMA-3 family on the generic Transformer (reference: example/llama3/config.h)."""
from __future__ import annotations

from ..nn.transformer import TransformerConfig, TransformerModel

_SIZES = {
    "llama3-1b": dict(n_layer=16, n_embd=2048, n_head=32, n_kv_head=8, ffn_dim_multiplier=1.5, multiple_of=256),
    "llama3-3b": dict(n_layer=28, n_embd=3072, n_head=24, n_kv_head=8, ffn_dim_multiplier=1.0, multiple_of=256),
    "llama3-8b": dict(n_layer=32, n_embd=4096, n_head=32, n_kv_head=8, ffn_dim_multiplier=1.3, multiple_of=1024),
}


def llama3_config(name: str = "llama3-1b", **overrides) -> TransformerConfig:
    kw = dict(_SIZES[name])
    kw.update(overrides)
    return TransformerConfig.LLaMA3(**kw)


def LLaMA3(name: str = "llama3-1b", **overrides) -> TransformerModel:
    return TransformerModel(llama3_config(name, **overrides))
