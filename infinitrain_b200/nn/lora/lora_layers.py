"""LoRA layers: plain, column-parallel and row-parallel linears with a low-rank update.

Reference: infini_train/src/nn/lora/lora_linear.cc:52-153, lora_parallel_linear.cc:91-203,288-403.
``y = base(x) + (alpha / r) * (x A^T) B^T`` with A ``[r, in]`` (Kaiming-uniform) and B ``[out, r]``
(zeros).  Under tensor parallelism the column-parallel variant replicates A and shards B along the
output dimension; the row-parallel variant shards A along the input dimension and replicates B, and
its low-rank product is reduced together with the base output.  ``MergeWeights`` folds
``(alpha / r) * B @ A`` into the base weight and freezes A / B; calling ``Forward`` on a merged layer
whose adapter still requires grad is an error, as in the reference.
"""
from __future__ import annotations

import math

import torch

from ...ops import functional as ops
from ...parallel import global_env as genv
from ...parallel import tensor_parallel as tpmod
from ...parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from .. import init
from ..layers import Linear
from ..module import Module
from .lora_config import LoRAConfig


def _init_ab(A, B, config: LoRAConfig, generator=None, a_full_shape=None, a_cols=None):
    """``generator``: where A is drawn from (None: the global stream).  With ``a_full_shape`` the draw has
    that shape (the factor of the unsharded layer) and ``a_cols = (begin, end)`` names this rank's columns."""
    target = A if a_full_shape is None else torch.empty(a_full_shape, dtype=torch.float32)
    if config.use_kaiming_a:
        init.KaimingUniform(target, a=config.kaiming_a_param, generator=generator)
    else:
        init.Normal(target, 0.0, 0.02, generator=generator)
    if target is not A:
        with torch.no_grad():
            A.copy_(target[:, a_cols[0]:a_cols[1]].to(A.dtype))
    init.Zeros(B)


class _LoRAMixin:
    """Shared bookkeeping: adapter parameters, merge state, freezing of the base."""

    kParamLoraAName = "lora_A"
    kParamLoraBName = "lora_B"

    def _setup_lora(self, config: LoRAConfig, a_shape, b_shape, device, generator=None, a_full_shape=None, a_cols=None):
        self.config = config
        self.merged_ = False
        self.lora_A = torch.nn.Parameter(torch.empty(a_shape, device=device))
        self.lora_B = torch.nn.Parameter(torch.empty(b_shape, device=device))
        _init_ab(self.lora_A, self.lora_B, config, generator, a_full_shape, a_cols)
        self.weight.requires_grad_(False)
        if getattr(self, "bias", None) is not None:
            self.bias.requires_grad_(False)

    def scaling(self) -> float:
        return self.config.Scaling()

    def rank(self) -> int:
        return self.config.rank

    def IsMerged(self) -> bool:
        return self.merged_

    def LoRAParameters(self):
        return [self.lora_A, self.lora_B]

    def _check_forward_allowed(self):
        if self.merged_ and (self.lora_A.requires_grad or self.lora_B.requires_grad):
            raise RuntimeError("Forward() on merged LoRA with requires_grad=true. Call UnmergeWeights() before training.")

    def _delta(self):
        return (self.lora_B.detach().float() @ self.lora_A.detach().float()) * self.config.Scaling()

    def MergeWeights(self):
        if self.merged_:
            return
        with torch.no_grad():
            self.weight.add_(self._delta().to(self.weight.dtype))
        self.merged_ = True
        self.lora_A.requires_grad_(False)
        self.lora_B.requires_grad_(False)

    def UnmergeWeights(self):
        if not self.merged_:
            return
        with torch.no_grad():
            self.weight.sub_(self._delta().to(self.weight.dtype))
        self.merged_ = False
        self.lora_A.requires_grad_(True)
        self.lora_B.requires_grad_(True)

    def _lora_path(self, x):
        """(alpha / r) * (x A^T) B^T through the same fused linear op as the base layer."""
        h = ops.linear(x, self.lora_A)
        return ops.linear(h, self.lora_B) * self.config.Scaling()


class LoRALinear(_LoRAMixin, Linear):
    kType = "LoRALinear"

    def __init__(self, in_features=None, out_features=None, config: LoRAConfig = None, bias: bool = True, device=None,
                 base_module: Linear = None, generator=None):
        if base_module is not None:
            Module.__init__(self, self.kType)
            self.in_features, self.out_features = base_module.in_features, base_module.out_features
            self.weight, self.bias = base_module.weight, base_module.bias
            device = self.weight.device
        else:
            Linear.__init__(self, in_features, out_features, bias, device)
            self._type = self.kType
        self._setup_lora(config or LoRAConfig(), (config.rank, self.in_features), (self.out_features, config.rank), device,
                         generator)

    def Forward(self, x):
        self._check_forward_allowed()
        y = ops.linear(x, self.weight, self.bias)
        if self.merged_:
            return y
        return y + self._lora_path(x).to(y.dtype)


class LoRAColumnParallelLinear(_LoRAMixin, ColumnParallelLinear):
    """A replicated ``[r, in]``, B sharded ``[out / tp, r]``."""

    kType = "LoRAColumnParallelLinear"

    def __init__(self, base_module: ColumnParallelLinear, config: LoRAConfig, generator=None):
        Module.__init__(self, self.kType)
        for k in ("in_features", "out_features", "output_size_per_partition", "has_bias", "gather_output",
                  "input_is_parallel", "skip_bias_add", "sequence_parallel"):
            setattr(self, k, getattr(base_module, k))
        self.weight, self.bias = base_module.weight, base_module.bias
        self._setup_lora(config, (config.rank, self.in_features), (self.output_size_per_partition, config.rank),
                         self.weight.device, generator)
        # A is replicated but every rank back-propagates through its own shard of B: each holds one
        # term of A's gradient, with or without sequence parallelism; the terms are summed over the
        # tensor-parallel group before the optimizer step.
        self.lora_A._itb_tp_partial_grad = True

    def Forward(self, x, gelu: bool = False):
        self._check_forward_allowed()
        add_bias = self.bias if (self.has_bias and not self.skip_bias_add) else None
        if self.sequence_parallel:
            xin = tpmod.GatherFromSPRegionFunc(x)
        elif not self.input_is_parallel:
            xin = tpmod.CopyToTPRegionFunc(x)
        else:
            xin = x
        y = ops.linear(xin, self.weight, add_bias)
        if not self.merged_:
            y = y + self._lora_path(xin).to(y.dtype)
        if gelu:
            y = ops.gelu(y)
        if self.gather_output:
            y = tpmod.GatherFromTPRegionFunc(y)
        if self.skip_bias_add:
            return y, self.bias
        return y


class LoRARowParallelLinear(_LoRAMixin, RowParallelLinear):
    """A sharded ``[r, in / tp]``, B replicated ``[out, r]``."""

    kType = "LoRARowParallelLinear"

    def __init__(self, base_module: RowParallelLinear, config: LoRAConfig, generator=None):
        Module.__init__(self, self.kType)
        for k in ("in_features", "out_features", "input_size_per_partition", "has_bias", "reduce_output",
                  "input_is_parallel", "skip_bias_add", "sequence_parallel"):
            setattr(self, k, getattr(base_module, k))
        self.weight, self.bias = base_module.weight, base_module.bias
        full, cols = None, None
        if generator is not None and self.input_size_per_partition != self.in_features:
            # a layout-independent start: the unsharded factor is drawn, this rank keeps its columns
            from ...parallel import global_env as genv

            r = genv.GetTensorParallelRank()
            full = (config.rank, self.in_features)
            cols = (r * self.input_size_per_partition, (r + 1) * self.input_size_per_partition)
        self._setup_lora(config, (config.rank, self.input_size_per_partition), (self.out_features, config.rank),
                         self.weight.device, generator, full, cols)
        # B is replicated but multiplies this rank's partial product x_r A_r^T: its gradient is one term
        # of a sum over the tensor-parallel group
        self.lora_B._itb_tp_partial_grad = True

    def Forward(self, x, residual=None):
        self._check_forward_allowed()
        if not self.input_is_parallel:
            x = tpmod.ScatterToTPRegionFunc(x)
        y = ops.linear(x, self.weight, None)
        if not self.merged_:
            # x A^T is a partial sum over the sharded input; B is linear, so reducing after B is the
            # same as reducing before it and shares the collective of the base output.
            y = y + self._lora_path(x).to(y.dtype)
        if self.reduce_output and tpmod._tp() is not None:
            y = tpmod.ReduceScatterToSPRegionFunc(y) if self.sequence_parallel else tpmod.ReduceFromTPRegionFunc(y)
        if self.has_bias and not self.skip_bias_add:
            y = y + self.bias.to(y.dtype)
        if residual is not None:
            y = y + residual
        if self.skip_bias_add:
            return y, self.bias
        return y
