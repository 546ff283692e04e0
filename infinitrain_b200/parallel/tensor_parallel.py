"""Tensor and sequence parallelism (Megatron style).

Reference: infini_train/src/nn/parallel/tensor_parallel.cc — region functions :133-232,
ColumnParallelLinear :270-315, RowParallelLinear :324-370, VocabParallelEmbedding :379-434,
VocabParallelCrossEntropy :436-572.

Activations are ``[B, T, C]``.  Under sequence parallelism the tensors between blocks are sharded
along T across the tensor-parallel group: an all-gather precedes every column-parallel linear and a
reduce-scatter follows every row-parallel linear (and the embedding).  The reference transposes to
put T first around every collective; here the gather / scatter are done along dim 1 directly, which
costs nothing when B == 1 and one strided copy otherwise.  On GPUs the all-gather + GEMM and
GEMM + reduce-scatter pairs have fused kernels in :mod:`infinitrain_b200.parallel.symm`; the
functions here are the NCCL / gloo formulation that every rank count and backend supports.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..nn import init
from ..nn.module import Module
from ..ops import functional as ops
from . import global_env as genv
from .process_group import ProcessGroup, ReduceOpType, tp_group


def _seq_dim(x: torch.Tensor) -> int:
    return 1 if x.dim() >= 3 else 0


def _tp() -> Optional[ProcessGroup]:
    g = tp_group()
    return g if (g is not None and g.world_size > 1) else None


# --------------------------------------------------------------------------- raw collectives
def _all_reduce(x: torch.Tensor, g: ProcessGroup) -> torch.Tensor:
    x = x.contiguous()
    g.AllReduce(x, ReduceOpType.kSum)
    return x


def _gather_along(x: torch.Tensor, g: ProcessGroup, dim: int) -> torch.Tensor:
    n = g.world_size
    x = x.contiguous()
    out = torch.empty((n,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    g.AllGather(out.view(-1), x.view(-1))
    if dim == 0:
        return out.view((n * x.shape[0],) + tuple(x.shape[1:]))
    # [n, d0, ..., d_dim, ...] -> [d0, ..., n * d_dim, ...]
    out = out.movedim(0, dim)
    shape = list(x.shape)
    shape[dim] *= n
    return out.reshape(shape)


def _reduce_scatter_along(x: torch.Tensor, g: ProcessGroup, dim: int) -> torch.Tensor:
    n = g.world_size
    shape = list(x.shape)
    assert shape[dim] % n == 0, "reduce-scatter dimension must divide by the group size"
    if dim != 0:
        # [..., n * s, ...] -> [n, ..., s, ...] so that rank r's shard is contiguous block r
        x = x.reshape(shape[:dim] + [n, shape[dim] // n] + shape[dim + 1:]).movedim(dim, 0)
    x = x.contiguous()
    shape[dim] //= n
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    g.ReduceScatter(out.view(-1), x.view(-1), ReduceOpType.kSum)
    return out


def _split_along_last(x: torch.Tensor, g: ProcessGroup) -> torch.Tensor:
    n, r = g.world_size, g.MyGroupRank()
    return x.chunk(n, dim=-1)[r].contiguous()


def _split_along(x: torch.Tensor, g: ProcessGroup, dim: int) -> torch.Tensor:
    n, r = g.world_size, g.MyGroupRank()
    return x.chunk(n, dim=dim)[r].contiguous()


# --------------------------------------------------------------------------- region functions
class CopyToTPRegion(torch.autograd.Function):
    """Identity forward, all-reduce of the gradient backward."""

    @staticmethod
    def forward(ctx, x):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        grp = _tp()
        return _all_reduce(g, grp) if grp else g


class ReduceFromTPRegion(torch.autograd.Function):
    """All-reduce forward, identity backward."""

    @staticmethod
    def forward(ctx, x):
        grp = _tp()
        return _all_reduce(x.clone(), grp) if grp else x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g


class ScatterToTPRegion(torch.autograd.Function):
    """Keep this rank's slice of the last dimension forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x):
        grp = _tp()
        return _split_along_last(x, grp) if grp else x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        grp = _tp()
        return _gather_along(g, grp, g.dim() - 1) if grp else g


class GatherFromTPRegion(torch.autograd.Function):
    """All-gather along the last dimension forward, slice backward."""

    @staticmethod
    def forward(ctx, x):
        grp = _tp()
        return _gather_along(x, grp, x.dim() - 1) if grp else x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        grp = _tp()
        return _split_along_last(g, grp) if grp else g


class ReduceScatterToSPRegion(torch.autograd.Function):
    """Reduce-scatter along the sequence dimension forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x):
        grp = _tp()
        ctx.dim = _seq_dim(x)
        return _reduce_scatter_along(x, grp, ctx.dim) if grp else x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        grp = _tp()
        return _gather_along(g, grp, ctx.dim) if grp else g


class GatherFromSPRegion(torch.autograd.Function):
    """All-gather along the sequence dimension forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x):
        grp = _tp()
        ctx.dim = _seq_dim(x)
        return _gather_along(x, grp, ctx.dim) if grp else x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        grp = _tp()
        return _reduce_scatter_along(g, grp, ctx.dim) if grp else g


def CopyToTPRegionFunc(x): return CopyToTPRegion.apply(x)
def ReduceFromTPRegionFunc(x): return ReduceFromTPRegion.apply(x)
def ScatterToTPRegionFunc(x): return ScatterToTPRegion.apply(x)
def GatherFromTPRegionFunc(x): return GatherFromTPRegion.apply(x)
def ReduceScatterToSPRegionFunc(x): return ReduceScatterToSPRegion.apply(x)
def GatherFromSPRegionFunc(x): return GatherFromSPRegion.apply(x)


def _linear_reset(weight, bias, fan_in):
    import math

    init.KaimingUniform(weight, a=math.sqrt(5.0))
    if bias is not None:
        bound = 1.0 / math.sqrt(fan_in) if fan_in > 0 else 0.0
        init.Uniform(bias, -bound, bound)


# --------------------------------------------------------------------------- layers
class ColumnParallelLinear(Module):
    """``y = x W^T + b`` with W split along the OUTPUT dimension: weight ``[out / tp, in]``."""

    kType = "ColumnParallelLinear"
    kParamWeightName = "weight"
    kParamBiasName = "bias"

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_output: bool = False,
                 input_is_parallel: bool = False, skip_bias_add: bool = False, sequence_parallel: bool = False,
                 device=None):
        super().__init__(self.kType)
        tp = genv.GetTensorParallelSize()
        if out_features % tp:
            raise ValueError("out_features must be divisible by the tensor-parallel size")
        self.in_features, self.out_features = in_features, out_features
        self.output_size_per_partition = out_features // tp
        self.has_bias, self.gather_output = bias, gather_output
        self.input_is_parallel, self.skip_bias_add = input_is_parallel, skip_bias_add
        self.sequence_parallel = sequence_parallel and tp > 1
        self.weight = torch.nn.Parameter(torch.empty(self.output_size_per_partition, in_features, device=device))
        self.bias = torch.nn.Parameter(torch.empty(self.output_size_per_partition, device=device)) if bias else None
        _linear_reset(self.weight, self.bias, in_features)

    def Forward(self, x, gelu: bool = False):
        from . import symm

        add_bias = self.bias if (self.has_bias and not self.skip_bias_add) else None
        if self.sequence_parallel and symm.fused_tp_enabled(x):
            symm.note_tp_path(self, x, True)
            y = symm.allgather_linear(x, self.weight, add_bias, gelu=gelu)
        elif (not self.sequence_parallel and not self.input_is_parallel and _tp() is not None
              and symm.fused_tp_enabled(x, seq_sharded=False)):
            # replicated input: no communication forward, the gradient all-reduce is fused into dgrad
            symm.note_tp_path(self, x, True)
            y = symm.copy_linear(x, self.weight, add_bias, gelu=gelu)
        else:
            if _tp() is not None:
                symm.note_tp_path(self, x, False)
            if self.sequence_parallel:
                x = GatherFromSPRegionFunc(x)
            elif not self.input_is_parallel:
                x = CopyToTPRegionFunc(x)
            y = ops.linear(x, self.weight, add_bias, gelu=gelu)
        if self.gather_output:
            y = GatherFromTPRegionFunc(y)
        if self.skip_bias_add:
            return y, self.bias
        return y


class RowParallelLinear(Module):
    """``y = x W^T + b`` with W split along the INPUT dimension: weight ``[out, in / tp]``."""

    kType = "RowParallelLinear"
    kParamWeightName = "weight"
    kParamBiasName = "bias"

    def __init__(self, in_features: int, out_features: int, bias: bool = True, reduce_output: bool = True,
                 input_is_parallel: bool = True, skip_bias_add: bool = False, sequence_parallel: bool = False,
                 device=None):
        super().__init__(self.kType)
        tp = genv.GetTensorParallelSize()
        if in_features % tp:
            raise ValueError("in_features must be divisible by the tensor-parallel size")
        if sequence_parallel and tp > 1 and not input_is_parallel:
            raise ValueError("To enable `sequence_parallel`, `input_is_parallel` must be `True`")
        self.in_features, self.out_features = in_features, out_features
        self.input_size_per_partition = in_features // tp
        self.has_bias, self.reduce_output = bias, reduce_output
        self.input_is_parallel, self.skip_bias_add = input_is_parallel, skip_bias_add
        self.sequence_parallel = sequence_parallel and tp > 1
        self.weight = torch.nn.Parameter(torch.empty(out_features, self.input_size_per_partition, device=device))
        self.bias = torch.nn.Parameter(torch.empty(out_features, device=device)) if bias else None
        _linear_reset(self.weight, self.bias, self.input_size_per_partition)

    def Forward(self, x, residual=None):
        """``residual`` (optional, already in the output's layout) is added after the reduction; with
        one tensor-parallel rank it is fused into the GEMM epilogue."""
        from . import symm

        if not self.input_is_parallel:
            x = ScatterToTPRegionFunc(x)
        add_bias = self.bias if (self.has_bias and not self.skip_bias_add) else None
        grp = _tp()
        if grp is None or not self.reduce_output:
            y = ops.linear(x, self.weight, add_bias, residual=residual)
        elif self.sequence_parallel and symm.fused_tp_enabled(x, seq_sharded=False):
            symm.note_tp_path(self, x, True)
            y = symm.linear_reduce_scatter(x, self.weight, add_bias, residual)
        elif not self.sequence_parallel and symm.fused_tp_enabled(x, seq_sharded=False):
            symm.note_tp_path(self, x, True)
            y = symm.linear_all_reduce(x, self.weight, add_bias, residual)
        else:
            symm.note_tp_path(self, x, False)
            y = ops.linear(x, self.weight, None)
            y = ReduceScatterToSPRegionFunc(y) if self.sequence_parallel else ReduceFromTPRegionFunc(y)
            if add_bias is not None:
                y = y + add_bias.to(y.dtype)
            if residual is not None:
                y = y + residual
        if self.skip_bias_add:
            return y, self.bias
        return y


class VocabParallelEmbedding(Module):
    """Embedding table split along the vocabulary: weight ``[V / tp, C]``; ids owned by other ranks
    contribute zero rows and the partial results are summed (all-reduce, or reduce-scatter along
    the sequence under sequence parallelism)."""

    kType = "VocabParallelEmbedding"
    kParamWeightName = "weight"

    def __init__(self, num_embeddings: int, embedding_dim: int, reduce_scatter_embeddings: bool = False, device=None):
        super().__init__(self.kType)
        tp = genv.GetTensorParallelSize()
        if num_embeddings % tp:
            raise ValueError("num_embeddings must be divisible by the tensor-parallel size")
        self.vocab_size_global = num_embeddings
        self.embedding_dim = embedding_dim
        self.reduce_scatter_embeddings = reduce_scatter_embeddings and tp > 1
        self.vocab_size_per_partition = num_embeddings // tp
        self.vocab_start_index = genv.GetTensorParallelRank() * self.vocab_size_per_partition
        self.vocab_end_index = self.vocab_start_index + self.vocab_size_per_partition
        self.weight = torch.nn.Parameter(torch.empty(self.vocab_size_per_partition, embedding_dim, device=device))
        init.Normal(self.weight)

    def Forward(self, tokens, wpe: Optional[torch.Tensor] = None, pos0: int = 0):
        """``wpe`` (optional position table) is fused into the lookup when there is one
        tensor-parallel rank; with several ranks the caller adds positions after the reduction."""
        grp = _tp()
        if grp is None:
            return ops.embedding(tokens, self.weight, wpe, pos0, 0)
        assert wpe is None, "position embedding is added after the tensor-parallel reduction"
        out = ops.embedding(tokens, self.weight, None, 0, self.vocab_start_index)
        return ReduceScatterToSPRegionFunc(out) if self.reduce_scatter_embeddings else ReduceFromTPRegionFunc(out)


class _VocabParallelCEFn(torch.autograd.Function):
    """Cross-entropy over logits sharded along the vocabulary, one collective.

    Each rank makes one pass over its ``[rows, V/tp]`` shard (local log-sum-exp and, where it owns the
    target column, the target logit), the per-row pairs are all-gathered, every rank merges them into
    the global log-sum-exp, and the backward pass rewrites the local shard in place with
    ``softmax_global - onehot``.  The reference issues ~20 elementwise launches and three
    all-reduces for the same result (tensor_parallel.cc:436-541).
    """

    @staticmethod
    def forward(ctx, logits, target, grp, vocab_valid_local, vocab_start):
        V_local = logits.shape[-1]
        l2 = logits.reshape(-1, V_local)
        rows = l2.shape[0]
        t_local = (target.reshape(-1) - vocab_start).contiguous()
        if l2.is_cuda:
            C = ops._C()
            if l2.stride(-1) != 1:
                l2 = l2.contiguous()
            _, lse_local, row_loss = C.ce_fwd(l2, t_local, vocab_valid_local)
        else:
            lv = l2[:, :vocab_valid_local].float()
            lse_local = torch.logsumexp(lv, dim=-1) if vocab_valid_local > 0 else torch.full((rows,), -1e30)
            own = (t_local >= 0) & (t_local < vocab_valid_local)
            picked = lv.gather(1, t_local.clamp(0, max(vocab_valid_local - 1, 0)).unsqueeze(1)).squeeze(1)
            row_loss = torch.where(own, lse_local - picked, torch.zeros_like(lse_local))
        if l2.is_cuda:
            from . import symm

            merge = symm.VocabCEMerge.get(l2.device)
            if merge is not None:
                # one kernel exchanges the per-row pairs over NVLink and merges them
                lse, loss_rows = merge(lse_local, row_loss, t_local, vocab_valid_local)
                ctx.save_for_backward(l2, t_local, lse)
                ctx.meta = (logits.shape, vocab_valid_local, rows)
                return loss_rows.view(target.shape)
        own = (t_local >= 0) & (t_local < vocab_valid_local)
        # target logit (0 where another rank owns it)
        tgt_logit = torch.where(own, lse_local - row_loss, torch.zeros_like(lse_local))
        stats = torch.stack([lse_local, tgt_logit], dim=0).contiguous()            # [2, rows]
        n = grp.world_size
        allst = torch.empty((n,) + tuple(stats.shape), dtype=stats.dtype, device=stats.device)
        grp.AllGather(allst.view(-1), stats.view(-1))
        lse = torch.logsumexp(allst[:, 0], dim=0)
        tgt = allst[:, 1].sum(0)
        loss_rows = lse - tgt
        ctx.save_for_backward(l2, t_local, lse)
        ctx.meta = (logits.shape, vocab_valid_local, rows)
        return loss_rows.view(target.shape)

    @staticmethod
    def backward(ctx, g):
        l2, t_local, lse = ctx.saved_tensors
        shape, vvalid, rows = ctx.meta
        g = g.reshape(-1).float()
        if l2.is_cuda:
            C = ops._C()
            # The kernel scales by (*grad_out) / rows with one scalar; per-row upstream gradients are
            # folded into the saved log-sum-exp: exp(x - lse + log g) = g * exp(x - lse) needs g > 0,
            # so scale afterwards instead when g is not uniform.
            one = torch.full((1,), float(rows), device=l2.device)
            C.ce_bwd(l2, t_local, lse.contiguous(), one, vvalid, False)
            grad = l2 * g.view(-1, 1).to(l2.dtype)
        else:
            lv = l2.float()
            p = torch.exp(lv - lse.view(-1, 1))
            p[:, vvalid:] = 0
            own = (t_local >= 0) & (t_local < vvalid)
            idx = t_local.clamp(0, max(vvalid - 1, 0))
            p[torch.arange(rows)[own], idx[own]] -= 1.0
            grad = (p * g.view(-1, 1)).to(l2.dtype)
        return grad.view(shape), None, None, None, None


class VocabParallelCrossEntropy:
    """Per-token loss over vocabulary-sharded logits (``Apply`` returns a ``[B, T]`` tensor)."""

    def __init__(self, vocab_size_original: int = 0, label_smoothing: float = 0.0):
        if not (0.0 <= label_smoothing < 1.0):
            raise ValueError("label_smoothing must be in [0, 1)")
        self.vocab_size_original = vocab_size_original
        self.label_smoothing = label_smoothing

    def Apply(self, logits, target):
        grp = _tp()
        tp = grp.world_size if grp else 1
        rank = grp.MyGroupRank() if grp else 0
        V_local = logits.shape[-1]
        V_global = V_local * tp
        V_orig = self.vocab_size_original or V_global
        if V_orig > V_global:
            raise ValueError("original vocab size must be <= padded vocab size")
        vocab_start = rank * V_local
        valid_local = max(0, min(V_local, V_orig - vocab_start))
        if self.label_smoothing > 0.0 or grp is None:
            return self._composed(logits, target, grp, vocab_start, valid_local, V_orig)
        return _VocabParallelCEFn.apply(logits, target, grp, valid_local, vocab_start)

    def _composed(self, logits, target, grp, vocab_start, valid_local, V_orig):
        """Reference formulation with three all-reduces; used for label smoothing and tp == 1."""
        lf = logits.float()
        V_local = lf.shape[-1]
        col = torch.arange(V_local, device=lf.device)
        valid = (col < valid_local).view(*([1] * (lf.dim() - 1)), V_local)
        masked = lf.masked_fill(~valid, float("-inf"))
        gmax = masked.max(-1).values
        if grp:
            gmax = gmax.detach().clone()
            grp.AllReduce(gmax, ReduceOpType.kMax)
        shifted = masked - gmax.detach().unsqueeze(-1)
        t_local = target - vocab_start
        own = (t_local >= 0) & (t_local < valid_local)
        sum_exp = shifted.exp().sum(-1)
        sum_exp = ReduceFromTPRegionFunc(sum_exp) if grp else sum_exp
        pred = shifted.gather(-1, t_local.clamp(0, max(V_local - 1, 0)).unsqueeze(-1)).squeeze(-1)
        pred = torch.where(own, pred, torch.zeros_like(pred))
        pred = ReduceFromTPRegionFunc(pred) if grp else pred
        log_sum_exp = sum_exp.log()
        loss = log_sum_exp - pred
        if self.label_smoothing > 0.0:
            ssum = torch.where(valid, shifted, torch.zeros_like(shifted)).sum(-1)
            ssum = ReduceFromTPRegionFunc(ssum) if grp else ssum
            mean_logp = ssum / float(V_orig) - log_sum_exp
            loss = loss * (1.0 - self.label_smoothing) - mean_logp * self.label_smoothing
        return loss


class VocabParallelCrossEntropyLoss(Module):
    """Mean of :class:`VocabParallelCrossEntropy` over all tokens."""

    kType = "VocabParallelCrossEntropyLoss"

    def __init__(self, vocab_size_original: int = 0, label_smoothing: float = 0.0):
        super().__init__(self.kType)
        self.vocab_size_original = vocab_size_original
        self.label_smoothing = label_smoothing

    def Forward(self, logits, target):
        per_tok = VocabParallelCrossEntropy(self.vocab_size_original, self.label_smoothing).Apply(logits, target)
        return per_tok.reshape(-1).mean()


def _needs_tp_grad_sum(p) -> bool:
    """Replicated parameters whose gradient is, on each tensor-parallel rank, one term of a sum: those
    that see a slice of the sequence under sequence parallelism (``_itb_sp_replicated``), and those that
    sit next to a sharded factor whatever the sequence layout (``_itb_tp_partial_grad``: the replicated
    LoRA factors of column- and row-parallel layers)."""
    return (getattr(p, "_itb_tp_partial_grad", False)
            or (getattr(p, "_itb_sp_replicated", False) and genv.GetSequenceParallelEnabled()))


def InstallSequenceParallelGradHooks(params) -> int:
    """Sums the gradient of every sequence-parallel-replicated parameter over the tensor-parallel
    group INSIDE backward (a tensor hook, before the gradient is accumulated).  Needed wherever
    the gradient is consumed before backward returns -- ZeRO reduce-scatters into shards and the fused
    reduce-scatter + AdamW kernels run as soon as a bucket is complete -- so that a sum after
    backward (``AllReduceSequenceParallelGrads``) would come too late; parameters hooked here are
    skipped by that function.  Returns the number of parameters hooked."""
    grp = _tp()
    if grp is None:
        return 0
    n = 0
    for p in params:
        if not _needs_tp_grad_sum(p) or getattr(p, "_itb_sp_hooked", False) or not p.requires_grad:
            continue

        def hook(g, _grp=grp):
            out = g.detach().clone(memory_format=torch.contiguous_format)
            _grp.AllReduce(out, ReduceOpType.kSum)
            return out

        p.register_hook(hook)
        p._itb_sp_hooked = True
        n += 1
    return n


def AllReduceSequenceParallelGrads(model: torch.nn.Module) -> int:
    """Sums, over the tensor-parallel group, the gradients of parameters that are replicated across
    TP ranks but see only a slice of the sequence under sequence parallelism (norm weights, position
    table, row-parallel biases, replicated LoRA factors; they carry ``_itb_sp_replicated``).  Call it
    after backward and before the optimizer step.  Returns the number of tensors reduced.

    The reference does not do this (its replicated parameters drift apart across TP ranks when
    sequence parallelism is on); without sequence parallelism every rank already holds the full
    gradient and nothing is done.
    """
    grp = _tp()
    if grp is None:
        return 0
    grads = []
    for p in model.parameters():
        if _needs_tp_grad_sum(p) and not getattr(p, "_itb_sp_hooked", False):
            g = p.grad if p.grad is not None else getattr(p, "main_grad", None)
            if g is not None:
                grads.append(g)
    if not grads:
        return 0
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    grp.AllReduce(flat, ReduceOpType.kSum)
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g))
        off += n
    return len(grads)
