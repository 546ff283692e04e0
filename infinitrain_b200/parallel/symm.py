"""Symmetric memory and the fused compute+collective kernels over NVLink / NVSwitch.

Every rank of a group allocates the same buffer through ``torch.distributed._symmetric_memory``
(CUDA VMM allocations exchanged between the processes, peer-mapped, plus an NVLS multicast mapping
when the switch supports it).  The hand-written kernels of ``csrc/comm`` then read and write peers
directly (loads / stores on peer pointers, ``multimem.ld_reduce`` / ``multimem.st`` on the multicast
pointer) and synchronise through flag words in symmetric memory with bounded waits.

Nothing in this module runs on CPU ranks: gloo tests exercise the NCCL/gloo formulation of the same
operations in :mod:`tensor_parallel` and :mod:`ddp`.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from .. import _ext
from ..ops import functional as ops
from .process_group import ProcessGroup

kFlagChannels = 65536    # flag slots [channel][8] int32 per rank (2 MB)


class StreamWork:
    """Completion handle of a kernel launched on a side stream."""

    def __init__(self, event: "torch.cuda.Event"):
        self.event = event

    def WaitNonBlocking(self) -> bool:
        torch.cuda.current_stream().wait_event(self.event)
        return True

    def WaitBlocking(self, timeout_s: float = 0.0) -> bool:
        self.event.synchronize()
        return True

    def IsCompleted(self) -> bool:
        return self.event.query()


class NvlinkContext:
    """Symmetric allocations, flag words, side stream and status word of one process group."""

    _by_group: Dict[str, "NvlinkContext"] = {}

    @classmethod
    def get(cls, pg: ProcessGroup, device: torch.device) -> "NvlinkContext":
        key = f"{pg.name}:{device}"
        if key not in cls._by_group:
            cls._by_group[key] = cls(pg, device)
        return cls._by_group[key]

    def __init__(self, pg: ProcessGroup, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        self._symm_mem = symm_mem
        self.pg = pg
        self.device = device
        self.rank = pg.MyGroupRank()
        self.world = pg.world_size
        self.C = _ext.load(required=True)
        if self.world > self.C.MAX_RANKS:
            raise ValueError(f"NVLink kernels support at most {self.C.MAX_RANKS} ranks per group")
        self._allocs: List[Tuple[torch.Tensor, object]] = []
        self.use_multimem = os.environ.get("ITB_NVLS", "1") == "1"
        self.flags = self.alloc(kFlagChannels * self.C.MAX_RANKS, torch.int32, device)
        self.flag_ptrs, _ = self.ptrs(self.flags)
        self.err = torch.zeros(4, dtype=torch.int32, device=device)
        self.stream = torch.cuda.Stream(device=device, priority=-1)
        self._next_channel = 0
        # Launch epochs live on the device (one counter per channel, advanced by the kernels), so a
        # captured CUDA graph can replay the collectives.
        self.epoch_ctr = torch.zeros(kFlagChannels, dtype=torch.int32, device=device)
        pg.Barrier()

    # ------------------------------------------------------------------ memory
    def alloc(self, n: int, dtype: torch.dtype, device=None) -> torch.Tensor:
        """A zero-filled symmetric tensor of ``n`` elements (collective over the group)."""
        t = self._symm_mem.empty(n, dtype=dtype, device=device or self.device)
        hdl = self._symm_mem.rendezvous(t, group=self.pg.pg)
        t.zero_()
        torch.cuda.synchronize(self.device)
        self._allocs.append((t, hdl))
        return t

    def handle_of(self, t: torch.Tensor):
        for base, hdl in self._allocs:
            lo = base.data_ptr()
            if lo <= t.data_ptr() < lo + base.numel() * base.element_size():
                return base, hdl
        raise KeyError("tensor is not in symmetric memory of this context")

    def ptrs(self, t: torch.Tensor) -> Tuple[List[int], int]:
        """(per-rank base pointers, multicast pointer or 0) of the allocation that holds ``t``."""
        base, hdl = self.handle_of(t)
        mc = int(hdl.multicast_ptr) if self.use_multimem else 0   # 0 when the switch offers no multicast
        return [int(p) for p in hdl.buffer_ptrs], mc

    def offset_of(self, t: torch.Tensor) -> int:
        base, _ = self.handle_of(t)
        return (t.data_ptr() - base.data_ptr()) // base.element_size()

    # ------------------------------------------------------------------ flags
    def reserve_channels(self, n: int) -> int:
        ch = self._next_channel
        if ch + n > kFlagChannels:
            raise RuntimeError("out of NVLink flag channels")
        self._next_channel += n
        return ch

    def status(self) -> int:
        return int(self.err.cpu()[0].item())

    # ------------------------------------------------------------------ launch helper
    def launch(self, fn) -> StreamWork:
        """Runs ``fn()`` (which launches a kernel) on the context's side stream, ordered after the
        work already queued on the current stream."""
        cur = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        self.stream.wait_event(ready)
        with torch.cuda.stream(self.stream):
            fn()
            done = torch.cuda.Event()
            done.record(self.stream)
        ops._counters["launches"] += 1
        return StreamWork(done)


class BucketAllReduce:
    """In-place all-reduce(avg) of slices of one symmetric fp32 gradient buffer (DDP buckets)."""

    def __init__(self, ctx: NvlinkContext, grad_buffer: torch.Tensor):
        self.ctx = ctx
        self.buf = grad_buffer
        self.ptrs, self.mc = ctx.ptrs(grad_buffer)
        self.base_off = ctx.offset_of(grad_buffer)
        self._channels: Dict[Tuple[int, int], int] = {}

    def __call__(self, contents: torch.Tensor):
        ctx = self.ctx
        off = self.base_off + (contents.data_ptr() - self.buf.data_ptr()) // 4
        n = contents.numel()
        if (off | n) & 3:
            return None   # misaligned bucket: the caller falls back to NCCL
        key = (off, n)
        if key not in self._channels:
            self._channels[key] = ctx.reserve_channels(ctx.C.MAX_COMM_BLOCKS)
        ch0 = self._channels[key]
        return ctx.launch(lambda: ctx.C.nvl_allreduce_scale(self.ptrs, self.mc, ctx.flag_ptrs, off, n, ctx.rank,
                                                            ctx.world, ch0, 0, 1.0 / ctx.world, ctx.err,
                                                            ctx.epoch_ctr))


class FusedZeroBucketStep:
    """Reduce-scatter + AdamW + parameter broadcast of one bucket in a single kernel."""

    def __init__(self, ctx: NvlinkContext, buffer, bucket, m: torch.Tensor, v: torch.Tensor):
        self.ctx = ctx
        self.g_ptrs, self.g_mc = ctx.ptrs(buffer.grad_buffer)
        self.p_ptrs, self.p_mc = ctx.ptrs(buffer.param_buffer)
        self.s_ptrs, self.s_mc = ctx.ptrs(buffer.shadow_buffer)
        if not (self.g_mc and self.p_mc and self.s_mc):
            self.g_mc = self.p_mc = self.s_mc = 0
        # the three buffers are separate allocations with equal layouts: one element offset
        self.off = ctx.offset_of(buffer.grad_buffer) + bucket.offset
        assert ctx.offset_of(buffer.param_buffer) == ctx.offset_of(buffer.grad_buffer) == ctx.offset_of(buffer.shadow_buffer)
        self.n = bucket.numel
        self.m, self.v = m, v
        self.ch0 = ctx.reserve_channels(ctx.C.MAX_COMM_BLOCKS)

    def __call__(self, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, dev_hyper=None):
        ctx = self.ctx
        return ctx.launch(lambda: ctx.C.nvl_rs_adamw_bcast(
            self.g_ptrs, self.g_mc, self.p_ptrs, self.p_mc, self.s_ptrs, self.s_mc, self.m, self.v, ctx.flag_ptrs,
            self.off, self.n, ctx.rank, ctx.world, self.ch0, 0, lr, b1, b2, eps, wd, bc1, bc2, grad_scale,
            ctx.err, ctx.epoch_ctr, dev_hyper))


def nvlink_available(pg: Optional[ProcessGroup], device: torch.device) -> bool:
    """The fused kernels need a CUDA group of 2..8 ranks on one NVLink domain (one node)."""
    if pg is None or pg.world_size < 2 or device.type != "cuda":
        return False
    if pg.backend != "nccl":
        return False
    if os.environ.get("ITB_DISABLE_NVLINK_KERNELS", "0") == "1":
        return False
    return pg.world_size <= 8


# --------------------------------------------------------------------------- tensor parallel (fused)
_TP_CTX = None


def fused_tp_enabled(x: torch.Tensor) -> bool:
    """True when the fused all-gather+GEMM / GEMM+reduce-scatter kernels should serve ``x``."""
    return bool(x.is_cuda and _TP_CTX is not None)


def allgather_linear(x, weight, bias, gelu=False):
    raise RuntimeError("fused tensor-parallel kernels are not initialised")


def linear_reduce_scatter(x, weight, bias, residual):
    raise RuntimeError("fused tensor-parallel kernels are not initialised")
