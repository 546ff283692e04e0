"""GPT-2 family on the generic Transformer (reference: example/gpt2/config.h, example/gpt2/main.cc)."""
from __future__ import annotations

from ..nn.transformer import TransformerConfig, TransformerModel
from ..parallel import global_env as genv

_SIZES = {
    "gpt2": dict(n_layer=12, n_head=12, n_embd=768),            # 124M
    "gpt2-medium": dict(n_layer=24, n_head=16, n_embd=1024),     # 350M
    "gpt2-large": dict(n_layer=36, n_head=20, n_embd=1280),      # 774M
    "gpt2-xl": dict(n_layer=48, n_head=25, n_embd=1600),         # 1558M
    "d12": dict(n_layer=12, n_head=12, n_embd=768),
    "d24": dict(n_layer=24, n_head=16, n_embd=1024),
    "d36": dict(n_layer=36, n_head=20, n_embd=1280),
    "d48": dict(n_layer=48, n_head=25, n_embd=1600),
}


def gpt2_config(name: str = "gpt2", **overrides) -> TransformerConfig:
    kw = dict(_SIZES[name])
    kw["n_kv_head"] = kw["n_head"]
    # The vocabulary is padded to 50304 only under tensor parallelism (so that it divides by the TP
    # size); the loss masks the padded columns.
    if genv.GetTensorParallelSize() > 1:
        kw["vocab_size"] = 50304
    kw.update(overrides)
    if "n_kv_head" not in overrides:
        kw["n_kv_head"] = kw["n_head"]
    return TransformerConfig.GPT2(**kw)


def GPT2(name: str = "gpt2", **overrides) -> TransformerModel:
    return TransformerModel(gpt2_config(name, **overrides))
