"""Transformer hyper-parameters (reference: infini_train/include/nn/modules/transformer/transformer_config.h:23-61)."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional

import torch


class AttentionType(enum.IntEnum):
    kStandard = 0   # learned absolute positions (GPT-2)
    kRoPE = 1       # rotary position embedding (LLaMA-3)


class MLPType(enum.IntEnum):
    kGELU = 0
    kSwiGLU = 1


class NormType(enum.IntEnum):
    kLayerNorm = 0
    kRMSNorm = 1


@dataclass
class TransformerConfig:
    block_size: int = 1024
    vocab_size: int = 50304
    original_vocab_size: int = 50257
    n_layer: int = 12
    n_head: int = 12
    n_kv_head: int = 12
    n_embd: int = 768

    attention_type: AttentionType = AttentionType.kStandard
    activation_type: MLPType = MLPType.kGELU
    norm_type: NormType = NormType.kLayerNorm

    add_bias_linear: bool = True
    add_bias_lm_head: bool = False
    tie_weights: bool = True

    ffn_expansion_ratio: float = 4.0
    ffn_dim_multiplier: Optional[float] = 1.5
    multiple_of: int = 256

    rope_theta: float = 500000.0
    use_scaled_rope: bool = False
    norm_eps: float = 1e-5

    use_kv: bool = False
    flash: bool = True                     # attention always runs the tiled online-softmax kernel
    max_gen_batch_size: int = 4

    # dtype of the residual stream under bf16 autocast: torch.bfloat16 keeps every activation in
    # bf16; torch.float32 reproduces the reference's fp32 residual stream.
    residual_dtype: torch.dtype = torch.bfloat16

    def UseGQA(self) -> bool:
        return self.n_kv_head < self.n_head

    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    def ffn_hidden(self) -> int:
        """MLP width (reference: infini_train/src/nn/modules/transformer/mlp.cc:24-38)."""
        h = int(self.n_embd * self.ffn_expansion_ratio)
        if self.activation_type == MLPType.kSwiGLU:
            h = int(2 * h) // 3
        if self.ffn_dim_multiplier is not None:
            h = int(round(h * self.ffn_dim_multiplier))
        return (h + self.multiple_of - 1) // self.multiple_of * self.multiple_of

    def GetChunkSize(self) -> int:
        return self.n_layer

    @staticmethod
    def GPT2(**kw) -> "TransformerConfig":
        """GPT-2 124M: 12 layers, 12 heads, 768 wide, learned positions, GELU MLP 4x, tied head."""
        cfg = dict(block_size=1024, vocab_size=50257, original_vocab_size=50257, n_layer=12, n_head=12, n_kv_head=12,
                   n_embd=768, attention_type=AttentionType.kStandard, activation_type=MLPType.kGELU,
                   norm_type=NormType.kLayerNorm, add_bias_linear=True, add_bias_lm_head=False, tie_weights=True,
                   ffn_expansion_ratio=4.0, ffn_dim_multiplier=None, multiple_of=1, norm_eps=1e-5)
        cfg.update(kw)
        return TransformerConfig(**cfg)

    @staticmethod
    def LLaMA3(**kw) -> "TransformerConfig":
        """LLaMA-3.2 1B shape by default: 16 layers, 2048 wide, 32 query / 8 KV heads, FFN 8192."""
        cfg = dict(block_size=8192, vocab_size=128256, original_vocab_size=128256, n_layer=16, n_head=32, n_kv_head=8,
                   n_embd=2048, attention_type=AttentionType.kRoPE, activation_type=MLPType.kSwiGLU,
                   norm_type=NormType.kRMSNorm, add_bias_linear=False, add_bias_lm_head=False, tie_weights=False,
                   ffn_expansion_ratio=4.0, ffn_dim_multiplier=1.5, multiple_of=256, rope_theta=500000.0,
                   norm_eps=1e-5)
        cfg.update(kw)
        return TransformerConfig(**cfg)

    @staticmethod
    def LLaMA3_8B(**kw) -> "TransformerConfig":
        """LLaMA-3 8B shape: 32 layers, 4096 wide, 32 query / 8 KV heads, FFN 14336."""
        cfg = dict(n_layer=32, n_embd=4096, n_head=32, n_kv_head=8, ffn_dim_multiplier=1.3, multiple_of=1024)
        cfg.update(kw)
        return TransformerConfig.LLaMA3(**cfg)
