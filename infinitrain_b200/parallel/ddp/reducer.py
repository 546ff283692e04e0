"""Bucketed gradient all-reduce for data parallelism without sharding (ZeRO-0).

Reference: infini_train/src/nn/parallel/ddp/reducer.cc — bucket assignment :56-139, bucket views
:262-300, ready marking and in-order launch :328-401, finalisation :403-438, one-time rebuild in the
observed ready order :212-247.

Each bucket owns one flat fp32 ``contents`` tensor; with ``gradient_as_bucket_view`` every
``param.grad`` (and ``param.main_grad``, into which the weight-gradient GEMM accumulates directly)
is a view of it, so a ready bucket is reduced in place with no packing copy.  A bucket is launched
as soon as all of its gradients are ready AND every earlier bucket has been launched, as an
asynchronous all-reduce(avg) that overlaps the rest of backward; ``FinalizeBackward`` makes the
compute stream wait for the outstanding reductions.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ...ops.functional import autograd_ready_hook
from ..process_group import ProcessGroup, ReduceOpType, Work
from .config import DistributedDataParallelConfig

kBytesPerMB = 1024 * 1024


def ComputeBucketAssignmentBySize(tensors: Sequence[torch.Tensor], bucket_size_limits: Sequence[int],
                                  tensor_indices: Optional[Sequence[int]] = None) -> List[List[int]]:
    """Groups tensor indices into buckets.

    Tensors are walked in ``tensor_indices`` order (default: reverse, close to the order gradients
    become ready).  Tensors of different (device, dtype) never share a bucket.  A bucket is closed
    once its bytes reach the current cap — so buckets exceed the cap by up to one tensor — and the
    cap advances along ``bucket_size_limits`` (first cap small so communication starts early).
    """
    assert len(tensors) > 0 and len(bucket_size_limits) > 0
    order = list(tensor_indices) if tensor_indices else list(reversed(range(len(tensors))))
    states: Dict[tuple, dict] = {}
    key_order = []
    out: List[List[int]] = []

    def flush(s):
        if s["cur"]:
            out.append(s["cur"])
            s["cur"] = []
            s["bytes"] = 0
            if s["limit"] + 1 < len(bucket_size_limits):
                s["limit"] += 1

    for idx in order:
        t = tensors[idx]
        key = (str(t.device), t.dtype)
        if key not in states:
            states[key] = {"cur": [], "bytes": 0, "limit": 0}
            key_order.append(key)
        s = states[key]
        s["cur"].append(idx)
        s["bytes"] += t.numel() * t.element_size()
        if s["bytes"] >= bucket_size_limits[s["limit"]]:
            flush(s)
    for key in key_order:
        flush(states[key])
    return out


@dataclass
class _Bucket:
    variable_indices: List[int]
    contents: torch.Tensor
    offsets: List[int]
    pending: int = 0
    work: Optional[Work] = None
    launched: bool = False


class Reducer:
    def __init__(self, params: Sequence[torch.nn.Parameter], bucket_indices: List[List[int]],
                 pg: Optional[ProcessGroup], config: Optional[DistributedDataParallelConfig] = None,
                 allreduce_fn: Optional[Callable[[torch.Tensor], Optional[Work]]] = None, flat_buffer=None):
        self.params = list(params)
        # With a flat ParamAndGradBuffer every bucket is a contiguous slice of its gradient buffer
        # (the buffer is laid out in the same reverse order the buckets are filled in), so the
        # fused optimizer and the reducer share one allocation.  The layout then fixes the order and
        # the one-time rebuild is skipped.
        self.flat_buffer = flat_buffer
        self.pg = pg
        self.config = config or DistributedDataParallelConfig()
        self.allreduce_fn = allreduce_fn   # optional override: the fused NVLink kernel
        self.status_ctx = None             # the NvlinkContext whose status word that kernel writes
        self.buckets: List[_Bucket] = []
        self.locator: Dict[int, tuple] = {}
        self.next_bucket = 0
        self.expect_hooks = False
        self.grad_ready_order: List[int] = []
        self.has_rebuilt = False
        self.need_rebuild = False
        self._index_of = {id(p): i for i, p in enumerate(self.params)}
        self._marked = set()
        self._hook_handles = []
        self.InitializeBuckets(bucket_indices)

    # ------------------------------------------------------------------ buckets
    def InitializeBuckets(self, bucket_indices: List[List[int]]):
        self.buckets = []
        self.locator = {}
        for b, idxs in enumerate(bucket_indices):
            if self.flat_buffer is not None:
                rng = [self.flat_buffer.param_index_map[id(self.params[i])] for i in idxs]
                start, end = min(r[0] for r in rng), max(r[1] for r in rng)
                assert end - start == sum(self.params[i].numel() for i in idxs), \
                    "bucket is not contiguous in the flat gradient buffer"
                contents = self.flat_buffer.grad_buffer[start:end]
                offs = []
                for j, i in enumerate(idxs):
                    offs.append(rng[j][0] - start)
                    self.locator[i] = (b, j)
                self.buckets.append(_Bucket(list(idxs), contents, offs))
                continue
            numel = sum(self.params[i].numel() for i in idxs)
            ref = self.params[idxs[0]]
            contents = torch.zeros(numel, dtype=ref.dtype, device=ref.device)
            offs, off = [], 0
            for j, i in enumerate(idxs):
                p = self.params[i]
                offs.append(off)
                self.locator[i] = (b, j)
                if self.config.gradient_as_bucket_view:
                    view = contents[off:off + p.numel()].view(p.shape)
                    if p.grad is not None:
                        view.copy_(p.grad)
                    p.grad = view
                    p.main_grad = view
                off += p.numel()
            self.buckets.append(_Bucket(list(idxs), contents, offs))

    def GetBucketTensors(self) -> List[List[torch.nn.Parameter]]:
        return [[self.params[i] for i in b.variable_indices] for b in self.buckets]

    def RebuildBuckets(self):
        """Re-bucket once, in the order gradients actually became ready in the first iteration."""
        if not self.grad_ready_order or self.flat_buffer is not None:
            return
        seen = set(self.grad_ready_order)
        full = list(self.grad_ready_order) + [i for i in range(len(self.params)) if i not in seen]
        limits = [self.config.first_bucket_cap_mb * kBytesPerMB, self.config.normal_bucket_cap_mb * kBytesPerMB]
        self.InitializeBuckets(ComputeBucketAssignmentBySize(self.params, limits, full))

    # ------------------------------------------------------------------ hooks
    def AttachHooksToParameters(self):
        for p in self.params:
            if not p.requires_grad:
                continue
            self._hook_handles.append(p.register_post_accumulate_grad_hook(autograd_ready_hook(self._on_grad)))
            p._itb_grad_ready_hooks = [self._on_grad]

    def _on_grad(self, p):
        self.MarkVariableReadyDense(self._index_of[id(p)])

    def PrepareForBackward(self):
        """Called after every forward: arms the pending counters; applies the one-time rebuild."""
        if self.need_rebuild and not self.has_rebuilt:
            self.RebuildBuckets()
            self.has_rebuilt = True
            self.need_rebuild = False
        self.RebindGradViews()
        self.next_bucket = 0
        self.expect_hooks = True
        self._marked = set()
        for b in self.buckets:
            b.pending = sum(1 for i in b.variable_indices if self.params[i].requires_grad)
            b.work = None
            b.launched = False
        if not self.has_rebuilt:
            self.grad_ready_order = []

    def RebindGradViews(self):
        """After ``ZeroGrad(set_to_none=True)`` the ``.grad`` views are gone: point them at the bucket
        again and clear the stale bucket memory (a fresh step starts from zero); gradients that
        micro-batches under ``no_sync`` accumulated in tensors of their own are carried into the
        bucket; views that are still bound are left alone."""
        if not self.config.gradient_as_bucket_view or self.flat_buffer is not None:
            return
        for bucket in self.buckets:
            ps = [self.params[i] for i in bucket.variable_indices]
            if all(p.grad is not None and p.grad.data_ptr() == bucket.contents.data_ptr() + off * p.element_size()
                   for p, off in zip(ps, bucket.offsets)):
                continue
            bucket.contents.zero_()
            for p, off in zip(ps, bucket.offsets):
                view = bucket.contents[off:off + p.numel()].view(p.shape)
                if p.grad is not None:
                    # gradients of earlier micro-batches, accumulated outside the bucket while the
                    # synchronisation was off (no_sync): they move into the bucket, they are not dropped
                    view.copy_(p.grad)
                p.grad = view
                p.main_grad = view

    def MarkVariableReadyDense(self, index: int):
        if not self.expect_hooks or index in self._marked:
            # A parameter is counted once per backward pass: weights whose gradient GEMM accumulates
            # straight into the bucket report from there, and autograd's accumulate hook may fire
            # for them again with an undefined gradient.
            return
        self._marked.add(index)
        if not self.has_rebuilt:
            self.grad_ready_order.append(index)
        b, j = self.locator[index]
        bucket = self.buckets[b]
        p = self.params[index]
        if not self.config.gradient_as_bucket_view and p.grad is not None:
            bucket.contents[bucket.offsets[j]:bucket.offsets[j] + p.numel()].copy_(p.grad.reshape(-1))
        bucket.pending -= 1
        while self.next_bucket < len(self.buckets) and self.buckets[self.next_bucket].pending <= 0:
            self.FinalizeBucketDense(self.next_bucket)
            self.next_bucket += 1
        if self.next_bucket == len(self.buckets):
            self.FinalizeBackward()

    def FinalizeBucketDense(self, b: int):
        bucket = self.buckets[b]
        if bucket.launched:
            return
        bucket.launched = True
        if self.allreduce_fn is not None:
            bucket.work = self.allreduce_fn(bucket.contents)
        elif self.pg is not None and self.pg.world_size > 1:
            bucket.work = self.pg.AllReduce(bucket.contents, ReduceOpType.kAvg, async_op=True)

    def FinalizeBackward(self):
        """All buckets are in flight: the compute stream waits for each; unpack when not a view."""
        self.expect_hooks = False
        for bucket in self.buckets:
            if bucket.work is not None:
                bucket.work.WaitNonBlocking()
                bucket.work = None
            if not self.config.gradient_as_bucket_view:
                for j, i in enumerate(bucket.variable_indices):
                    p = self.params[i]
                    if p.grad is not None:
                        p.grad.copy_(bucket.contents[bucket.offsets[j]:bucket.offsets[j] + p.numel()].view(p.shape))
        if not self.has_rebuilt:
            self.need_rebuild = True
        if self.status_ctx is not None:
            # a fused all-reduce that gave up on a peer left its bucket unreduced: the word as of the
            # previous backward is checked here without a host sync, this backward's copy is queued
            if not torch.cuda.is_current_stream_capturing():
                self.status_ctx.check(sync=False, what="fused gradient all-reduce")
            self.status_ctx.poll_status()

    def Flush(self):
        """Launches whatever has not been launched (parameters that received no gradient)."""
        if not self.expect_hooks:
            return
        while self.next_bucket < len(self.buckets):
            self.FinalizeBucketDense(self.next_bucket)
            self.next_bucket += 1
        self.FinalizeBackward()

    def zero_grads(self):
        for b in self.buckets:
            b.contents.zero_()
