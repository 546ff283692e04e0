"""DistributedDataParallel: the module wrapper that keeps gradients of data-parallel replicas equal.

Reference: infini_train/src/nn/parallel/ddp/distributed_data_parallel.cc (modes :40-65,
ZeRO buffers :68-123, ZeRO-2 bypass hook :126-165, forward :208-218).

Three modes, chosen by the configuration exactly as in the reference:
* ``gradient_bucketing_enabled=False``: one all-reduce(avg) per parameter, issued from its
  post-accumulate hook;
* ZeRO-0 (default): :class:`Reducer` — size-capped buckets reduced asynchronously during backward;
* ZeRO-1 / ZeRO-2: :class:`ParamAndGradBuffer` + bucket groups — gradients are reduce-scattered to
  the owner shard and :class:`DistributedOptimizer` updates the shard and all-gathers parameters.
  ZeRO-3 is not supported (nor is it in the reference).

Construction broadcasts rank 0's parameters so that replicas start identical.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ...nn.module import Module
from ...ops.functional import autograd_ready_hook
from .. import global_env as genv
from ..process_group import ProcessGroup, ProcessGroupFactory, ReduceOpType
from .config import DistributedDataParallelConfig
from .param_and_grad_buffer import ParamAndGradBuffer, ParamAndGradBucketGroup, PartitionBuckets
from .reducer import ComputeBucketAssignmentBySize, Reducer, kBytesPerMB


class DistributedDataParallel(Module):
    kType = "DistributedDataParallel"
    kModuleName = "module"

    def __init__(self, module: torch.nn.Module, rank=None, config: Optional[DistributedDataParallelConfig] = None,
                 process_group: Optional[ProcessGroup] = None, broadcast_parameters: bool = True):
        super().__init__(self.kType)
        self.add_module(self.kModuleName, module)
        self.config = config or DistributedDataParallelConfig()
        if self.config.zero_stage >= 3:
            raise NotImplementedError("ZeRO-3 (parameter partitioning) is not supported")
        self.pg = process_group if process_group is not None else ProcessGroupFactory.Instance().dp_group()
        self.dp_size = self.pg.world_size if self.pg is not None else 1
        self.reducer: Optional[Reducer] = None
        self.nvlink_ctx = None
        self.param_grad_buffers: List[ParamAndGradBuffer] = []
        self.bucket_groups: List[ParamAndGradBucketGroup] = []
        self.param_to_group = {}
        self._hook_handles = []
        params = [p for p in module.parameters() if p.requires_grad]
        self._params = params
        if broadcast_parameters and self.dp_size > 1:
            with torch.no_grad():
                for p in module.parameters():
                    self.pg.BroadCast(p.data, 0)
                for b in module.buffers():
                    if b.is_floating_point():
                        self.pg.BroadCast(b.data, 0)
        if not params:
            return
        if self.config.zero_stage >= 1:
            # ZeRO consumes gradients during backward (reduce-scatter into shards; with the fused kernels
            # also the optimizer step): the tensor-parallel sum of sequence-parallel-replicated parameters'
            # gradients has to happen before that, inside backward
            from ..tensor_parallel import InstallSequenceParallelGradHooks

            InstallSequenceParallelGradHooks(params)
            self._build_param_and_grad_buffers(params)
        elif self.config.gradient_bucketing_enabled:
            self._build_reducer(params)
        else:
            for p in params:
                self._hook_handles.append(p.register_post_accumulate_grad_hook(self._allreduce_hook))

    # ------------------------------------------------------------------ mode: per-parameter
    def _allreduce_hook(self, p):
        if self.dp_size > 1 and p.grad is not None and getattr(self, "_sync_enabled", True):
            self.pg.AllReduce(p.grad, ReduceOpType.kAvg, async_op=False)

    # ------------------------------------------------------------------ mode: reducer (ZeRO-0)
    def _build_reducer(self, params):
        limits = [self.config.first_bucket_cap_mb * kBytesPerMB, self.config.normal_bucket_cap_mb * kBytesPerMB]
        flat = None
        allreduce_fn = None
        if all(p.is_cuda and p.dtype == torch.float32 for p in params):
            # One flat fp32 parameter / gradient buffer (+ bf16 shadow) shared with the fused
            # optimizer; buckets are contiguous slices of it.
            ctx = self._nvlink_context(params[0].device)
            flat = ParamAndGradBuffer(params, self.pg, DistributedDataParallelConfig(zero_stage=0),
                                      allocator=ctx.alloc if ctx is not None else None)
            for p in params:
                p._itb_flat_buffer = flat
            self.param_grad_buffers = [flat]
            if ctx is not None:
                from .. import symm

                fused = symm.BucketAllReduce(ctx, flat.grad_buffer)

                def allreduce_fn(contents, fused=fused, pg=self.pg):
                    work = fused(contents)
                    return work if work is not None else pg.AllReduce(contents, ReduceOpType.kAvg, async_op=True)
        indices = ComputeBucketAssignmentBySize(params, limits)
        self.reducer = Reducer(params, indices, self.pg, self.config, allreduce_fn=allreduce_fn, flat_buffer=flat)
        if allreduce_fn is not None:
            self.reducer.status_ctx = self.nvlink_ctx
        self.reducer.AttachHooksToParameters()

    # ------------------------------------------------------------------ mode: ZeRO-1/2
    def _nvlink_context(self, device):
        """The symmetric-memory context of the data-parallel group, or None when the fused NVLink
        kernels are off or unavailable (CPU ranks, gloo, more than 8 ranks)."""
        if not self.config.use_fused_nvlink_kernels:
            return None
        from .. import symm

        if not symm.nvlink_available(self.pg, device):
            return None
        self.nvlink_ctx = symm.NvlinkContext.get(self.pg, device)
        return self.nvlink_ctx

    def _build_param_and_grad_buffers(self, params):
        ctx = self._nvlink_context(params[0].device) if all(p.is_cuda and p.dtype == torch.float32 for p in params) else None
        buf = ParamAndGradBuffer(params, self.pg, self.config, allocator=ctx.alloc if ctx is not None else None)
        self.param_grad_buffers = [buf]
        for p in params:
            p._itb_flat_buffer = buf
        self.bucket_groups = PartitionBuckets(self.param_grad_buffers, self.pg, self.config)
        for i, g in enumerate(self.bucket_groups):
            for pid, p in g.params.items():
                self.param_to_group[pid] = g
        # Parameter all-gathers are chained in forward order (reverse of the bucket order).
        for i in range(len(self.bucket_groups) - 1, 0, -1):
            self.bucket_groups[i].SetNextParamGatherBucketGroup(self.bucket_groups[i - 1])
        for p in params:
            if buf.zero2_temp_grads:
                g = self.param_to_group[id(p)]
                p._itb_main_grad_fn = (lambda g=g, p=p: g.full_grad_view(p))
                self._hook_handles.append(p.register_post_accumulate_grad_hook(autograd_ready_hook(self._zero2_hook)))
            else:
                self._hook_handles.append(p.register_post_accumulate_grad_hook(autograd_ready_hook(self._on_grad_ready)))
            p._itb_grad_ready_hooks = [self._on_grad_ready]

    def _zero2_hook(self, p):
        """ZeRO-2: move the freshly accumulated gradient into the bucket's temporary full buffer and
        drop ``param.grad`` so that no persistent full-size gradient exists."""
        g = self.param_to_group[id(p)]
        if p.grad is not None:
            g.AccumulateParamGrad(p, p.grad)
            p.grad = None
        g.RegisterGradReady(p)

    def _on_grad_ready(self, p):
        g = self.param_to_group.get(id(p))
        if g is not None:
            g.RegisterGradReady(p)

    # ------------------------------------------------------------------ gradient accumulation
    def no_sync(self):
        """Context in which backward passes only accumulate gradients locally (micro-batches before
        the last one); the synchronisation is armed again on exit."""
        ddp = self

        class _NoSync:
            def __enter__(self_inner):
                ddp._sync_enabled = False
                if ddp.reducer is not None:
                    ddp.reducer.expect_hooks = False
                for g in ddp.bucket_groups:
                    g.is_last_microbatch = False

            def __exit__(self_inner, *exc):
                ddp._sync_enabled = True
                for g in ddp.bucket_groups:
                    g.is_last_microbatch = True
                return False

        return _NoSync()

    # ------------------------------------------------------------------ forward
    def Forward(self, *inputs, **kwargs):
        out = self._modules[self.kModuleName](*inputs, **kwargs)
        if self.reducer is not None and torch.is_grad_enabled() and getattr(self, "_sync_enabled", True):
            self.reducer.PrepareForBackward()
        return out

    def Parameters(self):
        return list(self._modules[self.kModuleName].parameters())

    def StateDict(self):
        m = self._modules[self.kModuleName]
        return m.StateDict() if hasattr(m, "StateDict") else m.state_dict(keep_vars=True)

    def LoadStateDict(self, sd):
        m = self._modules[self.kModuleName]
        m.LoadStateDict(sd)
        for buf in self.param_grad_buffers:
            buf.refresh_shadow()

    def FinishGradSync(self):
        """Waits for every outstanding gradient collective (also launches those whose parameters
        received no gradient)."""
        if self.reducer is not None:
            self.reducer.Flush()
        for g in self.bucket_groups:
            g.FinishGradSync()
