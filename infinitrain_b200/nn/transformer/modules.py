"""The generic Transformer: attention, MLP, layer, pipeline-aware first stage / chunk / last stage
and the assembled model.

Reference: infini_train/src/nn/modules/transformer/{causal_self_attention,mlp,transformer}.cc.
Every linear is a tensor-parallel layer (they reduce to plain linears with one TP rank), the
state-dict keys are the reference's (``transformer.wte.weight``, ``transformer.h.<i>.attn.c_attn.weight``,
``lm_head.weight``; children named ``__pp*`` alias the same modules and are skipped).

What differs from the reference, by design:
* attention is the tiled online-softmax kernel on the packed QKV projection: no ``[B, H, T, T]``
  tensor, no head repetition for GQA, no host-built mask, RoPE applied in place;
* residual adds run in the epilogue of the row-parallel GEMMs, GELU in the epilogue of ``c_fc``;
* weights are tied by sharing ONE Parameter between ``wte`` and ``lm_head`` (when pp == 1).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ...ops import functional as ops
from ...ops import reference as ref
from ...parallel import global_env as genv
from ...parallel.pp.stage_info import GetStageInfo, StageInfo
from ...parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding, _tp)
from ..layers import Embedding, LayerNorm, ModuleDict, ModuleList, NewGELU, RMSNorm, SwiGLU
from ..module import Module, kPPChunkNamePrefix, kPPFirstStageName, kPPLastStageName
from .config import AttentionType, MLPType, NormType, TransformerConfig


def PrecomputeFreqsCis(head_dim: int, end: int, theta: float = 10000.0, use_scaled: bool = False, device=None):
    """``[end, head_dim / 2, 2]`` (cos, sin) table."""
    return ref.precompute_freqs_cis(head_dim, end, theta, device)


def _aligned() -> bool:
    """True while the precision checker records module outputs: every module then computes exactly
    what the reference's module of the same name computes (no residual add inside the projections,
    GELU as its own module, token and position tables looked up separately), so that the two
    frameworks' per-module logs and dumps line up.  Off, the fused formulations run."""
    global _CHECK_ENV
    if _CHECK_ENV is None:
        from ...utils.precision_checker import PrecisionCheckEnv

        _CHECK_ENV = PrecisionCheckEnv.Instance()
    return int(_CHECK_ENV.config.level) != 0


_CHECK_ENV = None


def _make_norm(config: TransformerConfig):
    if config.norm_type == NormType.kLayerNorm:
        n = LayerNorm(config.n_embd)
    else:
        n = RMSNorm(config.n_embd, config.norm_eps)
    # Under sequence parallelism every TP rank sees a different slice of the sequence, so the
    # gradients of these replicated parameters must be summed over the TP group.
    for p in n.parameters():
        p._itb_sp_replicated = True
    return n


class CausalSelfAttention(Module):
    kType = "CausalSelfAttention"
    kCAttnLayerName = "c_attn"
    kCProjLayerName = "c_proj"

    def __init__(self, config: TransformerConfig):
        super().__init__(self.kType)
        self.config = config
        tp = genv.GetTensorParallelSize()
        if config.n_embd % config.n_head:
            raise ValueError("n_embd must be divisible by n_head")
        if config.n_head % tp:
            raise ValueError("n_head must be divisible by the tensor-parallel size")
        self.n_head, self.n_embd = config.n_head, config.n_embd
        self.head_dim = config.n_embd // config.n_head
        self.local_n_head = self.n_head // tp
        if config.UseGQA():
            if config.n_head % config.n_kv_head or config.n_kv_head % tp:
                raise ValueError("n_kv_head must divide n_head and be divisible by the tensor-parallel size")
            self.n_kv_head = config.n_kv_head
        else:
            self.n_kv_head = self.n_head
        self.local_n_kv_head = self.n_kv_head // tp
        self.n_rep = self.n_head // self.n_kv_head
        sp = genv.GetSequenceParallelEnabled()
        qkv_dim = (self.n_head + 2 * self.n_kv_head) * self.head_dim
        self.c_attn = ColumnParallelLinear(self.n_embd, qkv_dim, bias=config.add_bias_linear, gather_output=False,
                                           input_is_parallel=False, skip_bias_add=False, sequence_parallel=sp)
        self.c_proj = RowParallelLinear(self.n_embd, self.n_embd, bias=config.add_bias_linear, reduce_output=True,
                                        input_is_parallel=True, skip_bias_add=False, sequence_parallel=sp)
        if sp and self.c_proj.bias is not None:
            self.c_proj.bias._itb_sp_replicated = True

    def Forward(self, x, freqs_cis=None, start_pos: int = 0, residual=None):
        qkv = self.c_attn(x)
        rope = freqs_cis if self.config.attention_type == AttentionType.kRoPE else None
        y = ops.attention_packed(qkv, self.local_n_head, self.local_n_kv_head, self.head_dim, rope, start_pos, True)
        return self.c_proj(y, residual=residual)


class MLP(Module):
    kType = "MLP"
    kCFcLayerName = "c_fc"
    kCFc2LayerName = "c_fc2"
    kCProjLayerName = "c_proj"

    def __init__(self, config: TransformerConfig):
        super().__init__(self.kType)
        self.config = config
        hidden = config.ffn_hidden()
        sp = genv.GetSequenceParallelEnabled()
        self.c_fc = ColumnParallelLinear(config.n_embd, hidden, bias=config.add_bias_linear, gather_output=False,
                                         input_is_parallel=False, skip_bias_add=False, sequence_parallel=sp)
        if config.activation_type == MLPType.kSwiGLU:
            self.c_fc2 = ColumnParallelLinear(config.n_embd, hidden, bias=config.add_bias_linear, gather_output=False,
                                              input_is_parallel=False, skip_bias_add=False, sequence_parallel=sp)
            self.silu = SwiGLU()
        else:
            self.gelu = NewGELU()
        self.c_proj = RowParallelLinear(hidden, config.n_embd, bias=config.add_bias_linear, reduce_output=True,
                                        input_is_parallel=True, skip_bias_add=False, sequence_parallel=sp)
        if sp and self.c_proj.bias is not None:
            self.c_proj.bias._itb_sp_replicated = True

    def _plain(self) -> bool:
        """True when the children are the stock TP layers on one TP rank (no LoRA wrapper, no hook):
        then the whole MLP is one fused autograd function."""
        return (_tp() is None and type(self.c_fc) is ColumnParallelLinear and type(self.c_proj) is RowParallelLinear
                and not self.c_fc._fwd_pre_hooks and not self.c_fc._fwd_post_hooks
                and not self.c_proj._fwd_pre_hooks and not self.c_proj._fwd_post_hooks)

    def Forward(self, x, residual=None):
        if self.config.activation_type == MLPType.kSwiGLU:
            x1 = self.c_fc(x)
            x2 = self.c_fc2(x)
            if _aligned():
                y = self.c_proj(x1 * self.silu(x2))
                return y if residual is None else y + residual
            return self.c_proj(ops.swiglu(x1, x2), residual=residual)
        if _aligned():
            y = self.c_proj(self.gelu(self.c_fc(x)))
            return y if residual is None else y + residual
        if self._plain() and x.is_cuda:
            return ops.mlp_gelu(x, self.c_fc.weight, self.c_fc.bias, self.c_proj.weight, self.c_proj.bias, residual)
        h = self.c_fc(x, gelu=True) if type(self.c_fc) is ColumnParallelLinear else ops.gelu(self.c_fc(x))
        return self.c_proj(h, residual=residual)


class TransformerLayer(Module):
    kType = "Layer"                      # the reference's type name (transformer.h:12)

    def __init__(self, config: TransformerConfig):
        super().__init__(self.kType)
        self.ln_1 = _make_norm(config)
        self.attn = CausalSelfAttention(config)
        self.ln_2 = _make_norm(config)
        self.mlp = MLP(config)

    def Forward(self, x, freqs_cis=None, start_pos: int = 0):
        if _aligned():
            x1 = x + self.attn(self.ln_1(x), freqs_cis, start_pos)
            return x1 + self.mlp(self.ln_2(x1))
        # the residual connection starts at the norm (its second output), so that backward adds the
        # skip's gradient inside the norm's backward kernel
        y, xs = self.ln_1(x, skip=True)
        x1 = self.attn(y, freqs_cis, start_pos, residual=xs)
        y, x1s = self.ln_2(x1, skip=True)
        return self.mlp(y, residual=x1s)


class TransformerFirstStage(Module):
    kType = "TransformerFirstStage"
    kWTELayerName = "wte"
    kWPELayerName = "wpe"

    def __init__(self, config: TransformerConfig):
        super().__init__(self.kType)
        self.config = config
        self.wte = VocabParallelEmbedding(config.vocab_size, config.n_embd, genv.GetSequenceParallelEnabled())
        if config.attention_type == AttentionType.kStandard:
            self.wpe = Embedding(config.block_size, config.n_embd)
            self.wpe.weight._itb_sp_replicated = True

    def Forward(self, idx):
        T = idx.shape[1]
        if T > self.config.block_size:
            raise ValueError(f"Cannot forward sequence of length {T}, block size is only {self.config.block_size}")
        has_pos = self.config.attention_type == AttentionType.kStandard
        if _tp() is None and has_pos and _aligned():
            x = self.wte(idx) + self.wpe(torch.arange(T, device=idx.device))
        elif _tp() is None:
            x = self.wte(idx, self.wpe.weight if has_pos else None, 0)
        else:
            x = self.wte(idx)
            if has_pos:
                t_local = x.shape[1]
                start = genv.GetTensorParallelRank() * t_local if genv.GetSequenceParallelEnabled() else 0
                x = x + self.wpe.weight[start:start + t_local].to(x.dtype)
        if ops.autocast_enabled() and x.is_floating_point() and x.dtype != self.config.residual_dtype and x.is_cuda:
            x = x.to(self.config.residual_dtype)
        return x


class TransformerChunk(Module):
    kType = "TransformerChunk"
    kHLayerName = "h"
    kFreqsCisName = "freqs_cis"

    def __init__(self, config: TransformerConfig, start_layer: int, end_layer: int):
        super().__init__(self.kType)
        self.config = config
        self.h = ModuleList([TransformerLayer(config) for _ in range(start_layer, end_layer)])
        self._freqs: Optional[torch.Tensor] = None

    def _freqs_for(self, device):
        if self._freqs is None or self._freqs.device != device:
            self._freqs = PrecomputeFreqsCis(self.config.head_dim(), self.config.block_size * 2, self.config.rope_theta,
                                             self.config.use_scaled_rope, device)
        return self._freqs

    def Forward(self, x):
        freqs = self._freqs_for(x.device) if self.config.attention_type == AttentionType.kRoPE else None
        for layer in self.h:
            x = layer(x, freqs, 0)
        return x


class TransformerLastStage(Module):
    kType = "TransformerLastStage"
    kLnFLayerName = "ln_f"
    kLMHeadLayerName = "lm_head"

    def __init__(self, config: TransformerConfig):
        super().__init__(self.kType)
        self.config = config
        self.ln_f = _make_norm(config)
        self.lm_head = ColumnParallelLinear(config.n_embd, config.vocab_size, bias=config.add_bias_lm_head,
                                            gather_output=False, input_is_parallel=False, skip_bias_add=False,
                                            sequence_parallel=genv.GetSequenceParallelEnabled())

    def Forward(self, x):
        return self.lm_head(self.ln_f(x))


class TransformerModel(Module):
    """GPT-2 or LLaMA-3 depending on ``config``; holds only the layers of this pipeline stage."""

    kType = "Transformer"                # the reference's type name (transformer.h:71)
    kTransformerModelName = "transformer"

    def __init__(self, config: TransformerConfig, pp_rank: Optional[int] = None):
        super().__init__(self.kType)
        self.config = config
        pp = genv.GetPipelineParallelSize()
        pp_rank = genv.GetPipelineParallelRank() if pp_rank is None else pp_rank
        vpp = genv.GetVirtualPipelineParallelSize()
        if config.n_layer < pp * vpp:
            raise ValueError(f"the model has {config.n_layer} layers: too few for {pp} pipeline stages x {vpp} chunks each")
        self.stage_info: StageInfo = GetStageInfo(config.n_layer, pp, pp_rank, genv.GetVirtualPipelineParallelSize())
        tp = genv.GetTensorParallelSize()
        if config.vocab_size % tp:
            raise ValueError("Vocab size should be divisible by TP world size")
        transformer = {}
        if self.stage_info.is_first_stage:
            first = TransformerFirstStage(config)
            self.add_module(kPPFirstStageName, first)
            transformer[TransformerFirstStage.kWTELayerName] = first.wte
            if config.attention_type == AttentionType.kStandard:
                transformer[TransformerFirstStage.kWPELayerName] = first.wpe
        layers: List[Module] = []
        self.num_chunks = len(self.stage_info.layer_ranges_per_chunk)
        for ci, (s, e) in enumerate(sorted(self.stage_info.layer_ranges_per_chunk)):
            chunk = TransformerChunk(config, s, e)
            self.add_module(kPPChunkNamePrefix + str(ci), chunk)
            layers += list(chunk.h)
        transformer[TransformerChunk.kHLayerName] = ModuleList(layers)
        if self.stage_info.is_last_stage:
            last = TransformerLastStage(config)
            self.add_module(kPPLastStageName, last)
            transformer[TransformerLastStage.kLnFLayerName] = last.ln_f
            self.add_module(TransformerLastStage.kLMHeadLayerName, last.lm_head)
        self.add_module(self.kTransformerModelName, ModuleDict(transformer))
        if config.tie_weights and pp == 1:
            # One Parameter object serves both the embedding lookup and the output projection.
            shared = self._modules[kPPLastStageName].lm_head.weight
            self._modules[kPPFirstStageName].wte.weight = shared
            # Two ops produce gradient for this tensor: both go through autograd so that the
            # parameter's grad-ready hook fires once, after the last contribution.
            shared._itb_shared = True

    # ------------------------------------------------------------------ pipeline pieces
    def first_stage(self):
        return self._modules.get(kPPFirstStageName)

    def last_stage(self):
        return self._modules.get(kPPLastStageName)

    def chunk(self, i: int):
        return self._modules[kPPChunkNamePrefix + str(i)]

    def Forward(self, idx):
        x = self._modules[kPPFirstStageName](idx)
        for ci in range(self.num_chunks):
            x = self._modules[kPPChunkNamePrefix + str(ci)](x)
        return self._modules[kPPLastStageName](x)
