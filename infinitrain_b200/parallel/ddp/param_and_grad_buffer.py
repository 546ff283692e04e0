"""Flat parameter / gradient buffers with Megatron-style buckets.

Reference: infini_train/src/nn/parallel/ddp/param_and_grad_buffer.cc (layout rules :425-531, bucket
group synchronisation :149-405).  Layout rules kept because they fix the message sizes:
parameters are packed in REVERSE order (the order gradients become ready), with sharding
(ZeRO >= 1) every parameter starts at a multiple of 64 elements, a bucket closes once it holds at
least ``bucket_size_in_elements`` elements and its end is padded to ``lcm(dp, 128)`` elements
(optionally also 2**16); rank r of the data-parallel group owns elements
``[r * len / dp, (r + 1) * len / dp)`` of every bucket.

On top of the reference's fp32 parameter and gradient buffers there is a bf16 shadow of the
parameter buffer: the copy the GEMMs read, written by the fused optimizer kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..process_group import ProcessGroup, ReduceOpType, Work
from .config import DistributedDataParallelConfig

kParamStartAlignElements = 64
kBucketEndAlignElements = 128


def _pad_to(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class FlatLayout:
    param_ranges: List[Tuple[int, int, int]]       # per parameter (input order): (start, end, bucket id)
    bucket_ranges: List[Tuple[int, int]]           # per bucket: (start, end) with padding
    bucket_numel_unpadded: List[int]
    numel: int
    numel_unpadded: int


def plan_flat_layout(numels: Sequence[int], dp_size: int = 1, shard: bool = False,
                     bucket_size_in_elements: int = 1_000_000, pad_for_busbw: bool = False,
                     align_params: Optional[bool] = None) -> FlatLayout:
    """Pure layout computation (testable without tensors)."""
    align = shard if align_params is None else align_params
    n = len(numels)
    ranges: List[Optional[Tuple[int, int, int]]] = [None] * n
    buckets, unpadded = [], []
    pstart = bstart = 0
    bucket_id = 0
    pend = 0
    open_params = 0

    def close(pend_):
        nonlocal bstart, bucket_id, open_params
        unpadded.append(pend_ - bstart)
        bend = pend_
        if shard:
            l = math.lcm(dp_size, kBucketEndAlignElements)
            if pad_for_busbw:
                l = math.lcm(l, 1 << 16)
            bend = _pad_to(pend_, l)
        buckets.append((bstart, bend))
        bstart = bend
        bucket_id += 1
        open_params = 0
        return bend

    for i in reversed(range(n)):
        if align:
            pstart = _pad_to(pstart, kParamStartAlignElements)
        pend = pstart + numels[i]
        ranges[i] = (pstart, pend, bucket_id)
        open_params += 1
        if pend - bstart >= bucket_size_in_elements:
            pstart = close(pend)
        else:
            pstart = pend
    if open_params:
        close(pend)
    total = buckets[-1][1] if buckets else 0
    return FlatLayout(ranges, buckets, unpadded, total, sum(unpadded))


class ParamAndGradBucket:
    def __init__(self, bucket_id: int, params, param_data, grad_data, shadow_data, offset: int, numel_unpadded: int,
                 param_offsets: Dict[int, Tuple[int, int]], gradient_scaling_factor: float = 1.0):
        self.bucket_id = bucket_id
        self.params = params
        self.param_data = param_data          # fp32 view of the flat parameter buffer
        self.grad_data = grad_data            # fp32 view of the flat gradient buffer (None under ZeRO-2)
        self.shadow_data = shadow_data        # bf16 view (None when there is no shadow)
        self.offset = offset
        self.numel_unpadded = numel_unpadded
        self.param_offsets = param_offsets    # id(param) -> (start, end) inside the bucket
        self.gradient_scaling_factor = gradient_scaling_factor

    @property
    def numel(self) -> int:
        return self.param_data.numel()

    def GetTensorLocInBucket(self, param):
        return self.param_offsets.get(id(param))

    def ScaleGradients(self, factor: float):
        if self.grad_data is not None and factor != 1.0:
            self.grad_data.mul_(factor)


class ParamAndGradBuffer:
    """One flat fp32 parameter buffer, one flat fp32 gradient buffer and one bf16 shadow buffer.

    Parameters are re-pointed into the parameter buffer (``param.data`` becomes a view) and
    ``param.grad`` / ``param.main_grad`` into the gradient buffer, so a whole bucket is one
    contiguous message and the optimizer update is one kernel launch.
    """

    def __init__(self, params: Sequence[torch.nn.Parameter], ddp_pg: Optional[ProcessGroup] = None,
                 config: Optional[DistributedDataParallelConfig] = None, with_shadow: Optional[bool] = None,
                 allocator: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None):
        self.config = config or DistributedDataParallelConfig()
        self.params = list(params)
        assert self.params, "ParamAndGradBuffer needs at least one parameter"
        self.ddp_pg = ddp_pg
        self.dp_size = ddp_pg.world_size if ddp_pg is not None else 1
        self.dp_rank = ddp_pg.MyGroupRank() if (ddp_pg is not None and ddp_pg.world_size > 1) else 0
        zero = self.config.zero_stage
        dev = self.params[0].device
        self.device = dev
        self.layout = plan_flat_layout([p.numel() for p in self.params], self.dp_size, shard=zero >= 1,
                                       bucket_size_in_elements=self.config.bucket_size_in_elements,
                                       pad_for_busbw=self.config.pad_buckets_for_high_nccl_busbw)
        alloc = allocator or (lambda n, dt, d: torch.zeros(n, dtype=dt, device=d))
        self.numel = self.layout.numel
        self.param_buffer = alloc(self.numel, torch.float32, dev)
        # ZeRO-2 keeps no persistent full gradient buffer: full-bucket buffers live only from the
        # first gradient of a bucket to the end of its reduce-scatter.
        # (The NVLink kernels read peers' gradients in place, so with them the buffer stays.)
        keep_full_grads = zero < 2 or allocator is not None
        self.grad_buffer = alloc(self.numel, torch.float32, dev) if keep_full_grads else None
        self.zero2_temp_grads = zero >= 2 and not keep_full_grads
        if with_shadow is None:
            with_shadow = dev.type == "cuda"
        self.shadow_buffer = alloc(self.numel, torch.bfloat16, dev) if with_shadow else None
        self.param_index_map: Dict[int, Tuple[int, int, int]] = {}
        per_bucket: List[List] = [[] for _ in self.layout.bucket_ranges]
        with torch.no_grad():
            for p, (s, e, b) in zip(self.params, self.layout.param_ranges):
                self.param_index_map[id(p)] = (s, e, b)
                view = self.param_buffer[s:e].view(p.shape)
                view.copy_(p.data)
                p.data = view
                if self.grad_buffer is not None:
                    g = self.grad_buffer[s:e].view(p.shape)
                    p.grad = g
                    p.main_grad = g
                if self.shadow_buffer is not None:
                    sh = self.shadow_buffer[s:e].view(p.shape)
                    sh.copy_(view)
                    p._itb_shadow = sh
                    p._itb_shadow_version = p._version
                per_bucket[b].append(p)
        self.buckets: List[ParamAndGradBucket] = []
        for b, (bs, be) in enumerate(self.layout.bucket_ranges):
            offs = {id(p): (self.param_index_map[id(p)][0] - bs, self.param_index_map[id(p)][1] - bs)
                    for p in per_bucket[b]}
            self.buckets.append(ParamAndGradBucket(
                b, per_bucket[b], self.param_buffer[bs:be],
                None if self.grad_buffer is None else self.grad_buffer[bs:be],
                None if self.shadow_buffer is None else self.shadow_buffer[bs:be],
                bs, self.layout.bucket_numel_unpadded[b], offs))

    # ------------------------------------------------------------------ helpers
    def shard_range(self, bucket: ParamAndGradBucket, rank: Optional[int] = None) -> Tuple[int, int]:
        """[start, end) of ``rank``'s shard inside ``bucket`` (bucket-relative)."""
        rank = self.dp_rank if rank is None else rank
        n = bucket.numel // self.dp_size
        return rank * n, (rank + 1) * n

    def mark_shadows_fresh(self):
        for p in self.params:
            if getattr(p, "_itb_shadow", None) is not None:
                p._itb_shadow_version = p._version

    def refresh_shadow(self):
        if self.shadow_buffer is None:
            return
        if self.param_buffer.is_cuda:
            from ... import _ext

            _ext.load().cast_into(self.param_buffer, self.shadow_buffer)
        else:
            self.shadow_buffer.copy_(self.param_buffer)
        self.mark_shadows_fresh()

    def zero_grads(self):
        if self.grad_buffer is not None:
            self.grad_buffer.zero_()

    def Reset(self):
        self.zero_grads()


class ParamAndGradBucketGroup:
    """Buckets whose gradients are synchronised together (one bucket per group, like the
    reference's default).  ``RegisterGradReady`` counts parameters; when every parameter of the group
    has its gradient the collective is launched asynchronously, overlapping the rest of backward.
    """

    def __init__(self, buffer: ParamAndGradBuffer, buckets: Sequence[ParamAndGradBucket],
                 collective_pg: Optional[ProcessGroup], config: DistributedDataParallelConfig):
        self.buffer = buffer
        self.buckets = list(buckets)
        self.pg = collective_pg
        self.config = config
        self.pg_size = collective_pg.world_size if collective_pg is not None else 1
        self.rank_in_pg = collective_pg.MyGroupRank() if (collective_pg is not None and self.pg_size > 1) else 0
        self.params = {id(p): p for b in self.buckets for p in b.params}
        self.param_to_bucket = {id(p): (b, i) for i, b in enumerate(self.buckets) for p in b.params}
        self.params_with_grad = set()
        self.grad_reduce_works: List[Optional[Work]] = []
        self.param_gather_works: List[Optional[Work]] = []
        self.grad_reduce_dispatched = False
        self.grad_sync_done = False          # set by FinishGradSync, cleared by Reset (once per step)
        self.param_gather_dispatched = False
        self.is_last_microbatch = True
        self.next_param_gather_group: Optional["ParamAndGradBucketGroup"] = None
        # ZeRO-2: persistent 1/dp gradient shard per bucket + temporary full-bucket buffers.
        self.grad_shard_buffers: List[Optional[torch.Tensor]] = [None] * len(self.buckets)
        self.temp_full_grad: List[Optional[torch.Tensor]] = [None] * len(self.buckets)
        self.zero2 = config.zero_stage >= 2 and buffer.grad_buffer is None
        # Fused NVLink path: one callable per bucket that performs reduce-scatter + optimizer update
        # + parameter broadcast, and a callable that returns the optimizer's hyper-parameters.
        self.fused_steps: Optional[list] = None
        self.fused_hyper_fn = None
        self.fused_updated = False
        if self.zero2:
            for i, b in enumerate(self.buckets):
                self.grad_shard_buffers[i] = torch.zeros(b.numel // self.pg_size, dtype=torch.float32,
                                                         device=buffer.device)

    # ------------------------------------------------------------------ state
    def Reset(self):
        self.params_with_grad.clear()
        self.grad_reduce_works.clear()
        self.param_gather_works.clear()
        self.is_last_microbatch = True
        self.grad_reduce_dispatched = False
        self.grad_sync_done = False
        self.param_gather_dispatched = False
        self.fused_updated = False
        if self.zero2:
            self.temp_full_grad = [None] * len(self.buckets)

    # ------------------------------------------------------------------ ZeRO-2 gradient stash
    def full_grad_view(self, param) -> torch.Tensor:
        """The slot of ``param`` in its bucket's temporary full gradient buffer (created zeroed on
        first use in a step)."""
        bucket, bi = self.param_to_bucket[id(param)]
        if self.temp_full_grad[bi] is None:
            self.temp_full_grad[bi] = torch.zeros(bucket.numel, dtype=torch.float32, device=self.buffer.device)
        s, e = bucket.param_offsets[id(param)]
        return self.temp_full_grad[bi][s:e].view(param.shape)

    def AccumulateParamGrad(self, param, grad, overwrite: bool = False, rate: float = 1.0):
        view = self.full_grad_view(param)
        if overwrite:
            view.copy_(grad)
        else:
            view.add_(grad, alpha=rate)

    def GetLocalGradShardBuffer(self, bucket_idx: int):
        return self.grad_shard_buffers[bucket_idx]

    # ------------------------------------------------------------------ gradient sync
    def RegisterGradReady(self, param):
        if not self.config.overlap_grad_reduce or not self.is_last_microbatch:
            return
        if id(param) not in self.params:
            return
        self.params_with_grad.add(id(param))
        if len(self.params_with_grad) == len(self.params):
            self.StartGradSync()

    def StartGradSync(self):
        if self.grad_reduce_dispatched:
            return
        op = ReduceOpType.kAvg if self.config.average_in_collective else ReduceOpType.kSum
        async_op = self.config.overlap_grad_reduce
        if self.fused_steps is not None and self.fused_hyper_fn is not None:
            for step, bucket in zip(self.fused_steps, self.buckets):
                self.grad_reduce_works.append(step(*self.fused_hyper_fn(self, bucket)))
            self.fused_updated = True
            self.grad_reduce_dispatched = True
            self.params_with_grad.clear()
            return
        for i, bucket in enumerate(self.buckets):
            if self.zero2:
                full = self.temp_full_grad[i]
                if full is None:
                    full = torch.zeros(bucket.numel, dtype=torch.float32, device=self.buffer.device)
                    self.temp_full_grad[i] = full
                if self.pg is None or self.pg_size == 1:
                    self.grad_shard_buffers[i].copy_(full)
                    self.grad_reduce_works.append(None)
                else:
                    self.grad_reduce_works.append(self.pg.ReduceScatter(self.grad_shard_buffers[i], full, op, async_op))
                continue
            bucket.ScaleGradients(bucket.gradient_scaling_factor)
            if self.pg is None or self.pg_size == 1:
                self.grad_reduce_works.append(None)
            elif self.config.zero_stage >= 1:
                s, e = self.buffer.shard_range(bucket, self.rank_in_pg)
                self.grad_reduce_works.append(self.pg.ReduceScatter(bucket.grad_data[s:e], bucket.grad_data, op, async_op))
            else:
                self.grad_reduce_works.append(self.pg.AllReduce(bucket.grad_data, op, async_op))
        self.grad_reduce_dispatched = True
        self.params_with_grad.clear()

    def FinishGradSync(self):
        if self.grad_sync_done:
            return   # already reduced this step: a second reduce-scatter would mix reduced and raw data
        if not self.grad_reduce_dispatched:
            self.StartGradSync()
        for w in self.grad_reduce_works:
            if w is not None:
                w.WaitNonBlocking()
        self.grad_reduce_works.clear()
        if self.zero2:
            self.temp_full_grad = [None] * len(self.buckets)
        self.grad_reduce_dispatched = False
        self.grad_sync_done = True

    # ------------------------------------------------------------------ parameter sync
    def StartParamSync(self, force_sync: bool = False):
        """All-gather every rank's updated shard into the full parameter buffer."""
        assert self.config.zero_stage >= 1
        if self.param_gather_dispatched:
            return
        async_op = self.config.overlap_param_gather and not force_sync
        for bucket in self.buckets:
            if self.pg is None or self.pg_size == 1:
                self.param_gather_works.append(None)
                continue
            s, e = self.buffer.shard_range(bucket, self.rank_in_pg)
            self.param_gather_works.append(self.pg.AllGather(bucket.param_data, bucket.param_data[s:e], async_op))
        self.param_gather_dispatched = True

    def FinishParamSync(self, skip_next_bucket_dispatch: bool = False):
        if not self.param_gather_dispatched:
            self.StartParamSync()
        for w in self.param_gather_works:
            if w is not None:
                w.WaitNonBlocking()
        self.param_gather_works.clear()
        self.param_gather_dispatched = False
        if self.next_param_gather_group is not None and not skip_next_bucket_dispatch:
            self.next_param_gather_group.StartParamSync()

    def SetNextParamGatherBucketGroup(self, nxt: Optional["ParamAndGradBucketGroup"]):
        self.next_param_gather_group = nxt


def PartitionBuckets(buffers: Sequence[ParamAndGradBuffer], collective_pg: Optional[ProcessGroup],
                     config: DistributedDataParallelConfig) -> List[ParamAndGradBucketGroup]:
    """One bucket per group (reference: param_and_grad_buffer.cc:703-711)."""
    groups = []
    for buf in buffers:
        for b in buf.buckets:
            groups.append(ParamAndGradBucketGroup(buf, [b], collective_pg, config))
    return groups
