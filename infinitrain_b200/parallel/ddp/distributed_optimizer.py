"""ZeRO-1 / ZeRO-2 optimizer: every data-parallel rank updates only its 1/dp shard.

Reference: infini_train/src/nn/parallel/ddp/distributed_optimizer.cc — shard pieces :34-92,
``Step = FinishGradSync -> base.Step -> StartParamSync -> FinishParamSync`` :125-137, ZeroGrad
:110-123, state dict :139-147.

The reference intersects every parameter with the rank's shard of every bucket and hands the
resulting "param pieces" to the base optimizer (one small kernel per piece).  A rank's shard of a
bucket is one contiguous range, so here the base optimizer gets ONE tensor per bucket shard: the
update of a shard is a single fused kernel launch, and the optimizer state (m, v) exists only for the
shard.  After the update the fp32 shards are all-gathered into the full parameter buffer and the
bf16 shadow is refreshed.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Sequence

import torch

from ...optim.optimizer import Optimizer, OptimizerCreator
from .distributed_data_parallel import DistributedDataParallel
from .param_and_grad_buffer import ParamAndGradBucketGroup, ParamAndGradBuffer


class DistributedOptimizer(Optimizer):
    def __init__(self, creator: OptimizerCreator, full_params: Sequence[torch.nn.Parameter], model_chunks,
                 ddp_world_size: Optional[int] = None, ddp_rank: Optional[int] = None):
        super().__init__(full_params)
        chunks = model_chunks if isinstance(model_chunks, (list, tuple)) else [model_chunks]
        self.bucket_groups: List[ParamAndGradBucketGroup] = []
        self.buffers: List[ParamAndGradBuffer] = []
        for ch in chunks:
            assert isinstance(ch, DistributedDataParallel), "model chunks must be DistributedDataParallel modules"
            assert ch.config.zero_stage >= 1, "DistributedOptimizer needs zero_stage >= 1"
            self.bucket_groups += ch.bucket_groups
            self.buffers += ch.param_grad_buffers
        self.shard_params: List[torch.nn.Parameter] = []
        self.shard_meta = []   # (group, bucket index in group, start, end)
        for g in self.bucket_groups:
            for bi, bucket in enumerate(g.buckets):
                s, e = g.buffer.shard_range(bucket, g.rank_in_pg)
                shard = torch.nn.Parameter(bucket.param_data[s:e], requires_grad=True)
                shard._itb_no_flatten = True   # already a slice of a flat buffer: update it in place
                if g.zero2:
                    shard.grad = g.grad_shard_buffers[bi]
                else:
                    shard.grad = bucket.grad_data[s:e]
                if bucket.shadow_data is not None:
                    shard._itb_shadow = bucket.shadow_data[s:e]
                self.shard_params.append(shard)
                self.shard_meta.append((g, bi, s, e))
        self.base_optimizer = creator(self.shard_params)
        self.fused = self._install_fused_steps(chunks)

    def _install_fused_steps(self, chunks) -> bool:
        """With the NVLink kernels, a bucket's reduce-scatter, its AdamW update and the broadcast of
        the updated weights are ONE kernel launched as soon as the bucket's gradients are ready, i.e.
        the optimizer step overlaps the rest of backward.  Needs an Adam base optimizer."""
        from ...optim.optimizer import Adam
        from .. import symm

        base = self.base_optimizer
        self._nvlink_ctxs = []
        if not isinstance(base, Adam) or not all(getattr(ch, "nvlink_ctx", None) is not None for ch in chunks):
            return False
        k = 0
        for ch in chunks:
            ctx = ch.nvlink_ctx
            if ctx not in self._nvlink_ctxs:
                self._nvlink_ctxs.append(ctx)
            for g in ch.bucket_groups:
                steps = []
                for bucket in g.buckets:
                    steps.append(symm.FusedZeroBucketStep(ctx, g.buffer, bucket, base.m[k], base.v[k]))
                    k += 1
                g.fused_steps = steps
                g.fused_hyper_fn = self._fused_hyper
        return True

    def _fused_hyper(self, group: Optional[ParamAndGradBucketGroup] = None, bucket=None):
        """Arguments of one fused bucket launch.  The kernel sums the ranks' gradients, so the scale it
        applies afterwards carries the data-parallel average (``average_in_collective``, the
        reference's ``kAvg``: ddp/param_and_grad_buffer.cc:286-292) and the bucket's own
        ``gradient_scaling_factor``, as the NCCL formulation does."""
        b = self.base_optimizer
        t = b.t + 1   # the step these launches belong to (Step() increments t afterwards)
        scale = 1.0
        if group is not None:
            if group.config.average_in_collective:
                scale /= max(group.pg_size, 1)
            if bucket is not None:
                scale *= bucket.gradient_scaling_factor
        return (b.learning_rate, b.beta1, b.beta2, b.eps, b.weight_decay, 1.0 - b.beta1 ** t, 1.0 - b.beta2 ** t, scale,
                b._dev_hyper())

    def ZeroGrad(self, set_to_none: bool = True) -> None:
        if self.fused:
            # the bucket kernels that run during backward read the step state: advance it now
            self.base_optimizer.PrepareStep()
        for buf in self.buffers:
            buf.zero_grads()
        for g in self.bucket_groups:
            g.Reset()
        for p in self.params:
            if getattr(p, "main_grad", None) is None:
                p.grad = None

    def StartGradSync(self):
        for g in self.bucket_groups:
            g.StartGradSync()

    def FinishGradSync(self):
        for g in self.bucket_groups:
            g.FinishGradSync()

    def StartParamSync(self, force_sync: bool = False):
        for g in self.bucket_groups:
            g.StartParamSync(force_sync)

    def FinishParamSync(self, skip_next_bucket_dispatch: bool = True):
        for g in self.bucket_groups:
            g.FinishParamSync(skip_next_bucket_dispatch)
        for buf in self.buffers:
            buf.refresh_shadow()

    def Step(self) -> None:
        self.FinishGradSync()
        if self.fused:
            # Every bucket was reduced, updated and broadcast by its fused kernel during backward.
            # A kernel that gave up on a peer skipped its reduction: look at the status word as of the
            # previous step (pinned mirror, no host sync) and queue this step's copy.
            capturing = torch.cuda.is_current_stream_capturing()
            for ctx in self._nvlink_ctxs:
                if not capturing:
                    ctx.check(sync=False, what="fused ZeRO step")
                ctx.poll_status()
            self.base_optimizer.t += 1
            self.base_optimizer._prepared = False
            for buf in self.buffers:
                buf.mark_shadows_fresh()
            return
        self.base_optimizer.Step()
        self.StartParamSync()
        self.FinishParamSync(skip_next_bucket_dispatch=True)

    def StateDict(self):
        return self.base_optimizer.StateDict()

    def LoadStateDict(self, state_dict):
        self.base_optimizer.LoadStateDict(state_dict)

