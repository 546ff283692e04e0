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
        # pinned host mirror of the status word, refreshed by poll_status() without a host sync
        self.err_host = torch.zeros(4, dtype=torch.int32).pin_memory()
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
        # no rank may write into a peer's copy before that peer has finished zeroing it
        self.pg.Barrier()
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
        """The status word, read with a synchronous copy (0 = every bounded wait so far was met)."""
        return int(self.err.cpu()[0].item())

    def poll_status(self) -> None:
        """Queues a copy of the status word into the pinned host mirror on the current stream: no
        host synchronisation, and capturable in a CUDA graph (every replay refreshes the mirror)."""
        self.err_host.copy_(self.err, non_blocking=True)

    def check(self, sync: bool = False, what: str = "NVLink collective") -> None:
        """Raises ``KernelTimeout`` when a fused collective gave up waiting for a peer.  With
        ``sync=False`` it looks at the host mirror, i.e. at the state of the last completed
        ``poll_status``; a kernel that timed out skipped its reduction, so training must not go on."""
        code = self.status() if sync else int(self.err_host[0])
        if code != 0:
            from ..utils.fault_tolerance import KernelTimeout

            raise KernelTimeout(f"{what} of group {self.pg.name}: a bounded device-side wait gave up "
                                f"(code {code}); gradients / shards of this step are not reduced")

    @classmethod
    def check_all(cls, sync: bool = False) -> None:
        for ctx in list(cls._by_group.values()):
            ctx.check(sync)

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
class _SymBuf:
    """A symmetric workspace of the fused tensor-parallel GEMMs with its arrival counters."""

    def __init__(self, tp: "TpFusedContext", numel: int):
        nvl = tp.nvl
        self.t = nvl.alloc(numel, torch.bfloat16)
        self.ptrs, self.mc = nvl.ptrs(self.t)
        blk = tp.reserve_flag_block()
        self.arrive_ptrs = [p + blk * 32 for p in tp.flag_ptrs]      # int32[8] per block
        self.my_arrive = self.arrive_ptrs[tp.rank]
        self.total = torch.zeros(1, dtype=torch.int32, device=nvl.device)   # advanced by the kernels
        self.last_use: Optional[int] = None
        # the local shard whose gathered copy the buffer holds (kept alive so that its address cannot
        # be handed to another tensor) and that tensor's version at the push
        self.content: Optional[Tuple[torch.Tensor, int]] = None

    def holds(self, x2: torch.Tensor) -> bool:
        """True when the last push into this buffer gathered exactly ``x2`` (same memory, unmodified)."""
        if self.content is None:
            return False
        src, ver = self.content
        return (src.data_ptr() == x2.data_ptr() and src.shape == x2.shape and src.stride() == x2.stride()
                and x2._version == ver and src._version == ver)


class TpFusedContext:
    """Workspaces, counters and launch bookkeeping of the all-gather+GEMM / GEMM+reduce-scatter
    kernels of one tensor-parallel group.  Every rank must issue the same sequence of launches."""

    kFlagBlocks = 64

    def __init__(self, nvl: NvlinkContext):
        self.nvl = nvl
        self.C = nvl.C
        self.rank, self.world = nvl.rank, nvl.world
        self.flags = nvl.alloc(self.kFlagBlocks * 8, torch.int32)
        self.flag_ptrs, _ = nvl.ptrs(self.flags)
        self._next_block = 1                     # block 0: `started`
        self.launch_ctr = torch.zeros(1, dtype=torch.int32, device=nvl.device)
        self.cta_done = torch.zeros(1, dtype=torch.int32, device=nvl.device)
        self.launch_index = 0
        self._bufs: Dict[Tuple[str, int], _SymBuf] = {}

    def reserve_flag_block(self) -> int:
        if self._next_block >= self.kFlagBlocks:
            raise RuntimeError("out of tensor-parallel flag blocks")
        self._next_block += 1
        return self._next_block - 1

    def buf(self, tag: str, numel: int) -> _SymBuf:
        key = (tag, numel)
        if key not in self._bufs:
            self._bufs[key] = _SymBuf(self, numel)      # collective: all ranks get here together
        return self._bufs[key]

    def _lag(self, b: _SymBuf) -> int:
        return (self.launch_index - b.last_use) if b.last_use is not None else (1 << 24)

    def launch(self, a, a_mn, b, b_mn, M, N, K, c, c2, bias, aux, flags, *, batch, T, push=None, push_src=None,
               gate=None, gate_includes=1, slab=None, rs_out=None, rs_bias=None, rs_residual=None, bcast=None):
        C = self.C
        mode = (C.TP_PUSH if push is not None else 0) | (C.TP_GATE_A if gate is not None else 0) | \
               (C.TP_SCATTER if slab is not None else 0) | (C.TP_BROADCAST if bcast is not None else 0)
        tp = {"mode": mode, "rank": self.rank, "world": self.world, "T": T, "Tl": T // self.world, "batch": batch,
              "started": self.flag_ptrs, "launch_ctr": self.launch_ctr, "cta_done": self.cta_done}
        if push is not None:
            tp.update(push_src=push_src, gather=push.ptrs, gather_mc=push.mc, push_arrive=push.arrive_ptrs,
                      push_total=push.total, push_lag=self._lag(push))
        if gate is not None:
            tp.update(gate_arrive=gate.my_arrive, gate_total=gate.total, gate_includes_this_launch=gate_includes)
        if slab is not None:
            tp.update(slab=slab.ptrs, rs_arrive=slab.arrive_ptrs, rs_total=slab.total, rs_lag=self._lag(slab),
                      rs_out=rs_out, rs_bias=rs_bias, rs_residual=rs_residual)
        if bcast is not None:
            tp.update(ar_out=bcast.ptrs, ar_mc=bcast.mc, ar_arrive=bcast.arrive_ptrs, ar_total=bcast.total,
                      ar_lag=self._lag(bcast))
        C.tp_gemm(a, a_mn, b, b_mn, M, N, K, c, c2, bias, aux, flags, tp, self.nvl.err)
        ops._counters["launches"] += 1
        for bf in (push, gate, slab, bcast):
            if bf is not None:
                bf.last_use = self.launch_index
        if push is not None:
            push.content = (push_src, push_src._version)
        self.launch_index += 1

    def wait_arrivals(self, b: _SymBuf):
        """Holds the current stream until every rank's push into ``b`` has landed."""
        self.C.tp_wait(b.my_arrive, b.total, self.world, self.nvl.err)
        ops._counters["launches"] += 1


_TP_CTX: Optional[TpFusedContext] = None
_TP_TRIED = False


def _tp_context(device: torch.device) -> Optional[TpFusedContext]:
    global _TP_CTX, _TP_TRIED
    if _TP_CTX is None and not _TP_TRIED:
        _TP_TRIED = True
        from .process_group import tp_group

        g = tp_group()
        if os.environ.get("ITB_FUSED_TP", "1") == "1" and nvlink_available(g, device):
            _TP_CTX = TpFusedContext(NvlinkContext.get(g, device))
    return _TP_CTX


def reset_fused_tp():
    """Forgets the context (tests that rebuild the process groups)."""
    global _TP_CTX, _TP_TRIED
    _TP_CTX, _TP_TRIED = None, False


# Which formulation the tensor-parallel linears ran: calls served by the fused all-gather+GEMM /
# GEMM+reduce-scatter kernels and calls that fell back to NCCL collectives around a plain GEMM.  A
# benchmark quotes these so that a "fused" number cannot come from the fallback unnoticed.
tp_path_counts: Dict[str, int] = {"fused": 0, "nccl": 0}
_tp_path_logged: set = set()


def note_tp_path(module, x: torch.Tensor, fused: bool) -> None:
    """Counts the call and logs, once per layer and path, which formulation served it."""
    tp_path_counts["fused" if fused else "nccl"] += 1
    key = (id(module), fused)
    if key in _tp_path_logged:
        return
    _tp_path_logged.add(key)
    if os.environ.get("ITB_LOG_TP_PATH", "0") == "1" or (not fused and x.is_cuda):
        from ..utils.logging import LOG

        why = "" if fused else (" (the fused kernels need a bf16 CUDA activation [B, T, C] with C % 8 == 0 and "
                                f"T / tp a multiple of {kTpRowTile}; got {tuple(x.shape)} {x.dtype})")
        LOG("INFO", f"{type(module).__name__}({getattr(module, 'in_features', '?')} -> "
                    f"{getattr(module, 'out_features', '?')}): "
                    f"{'fused NVLink kernel' if fused else 'NCCL collective + GEMM'}{why}")


kTpRowTile = 256     # rows of one output tile of the fused kernels: T / tp must be a multiple of it


def fused_tp_enabled(x: torch.Tensor, seq_sharded: bool = True) -> bool:
    """True when the fused all-gather+GEMM / GEMM+reduce-scatter kernels can serve ``x``: a 3-D CUDA
    activation under bf16 whose per-rank sequence length is a multiple of 256."""
    if not (x.is_cuda and x.dim() == 3 and ops._use_fused(x) and x.shape[-1] % 8 == 0):
        return False
    tp = _tp_context(x.device)
    if tp is None:
        return False
    t_local = x.shape[1] if seq_sharded else x.shape[1] // tp.world
    return t_local % kTpRowTile == 0 and (seq_sharded or x.shape[1] % tp.world == 0)


class _AllGatherLinearFn(torch.autograd.Function):
    """y[B, T, N] = all_gather_T(x[B, T/tp, K]) W^T (+ bias) (optionally GELU), one launch per rank.

    Backward: one launch computes dX = reduce_scatter_T(dY W) and re-gathers x for the weight
    gradient, which follows as a plain GEMM once the shards have arrived."""

    @staticmethod
    def forward(ctx, x, weight, bias, gelu):
        tp = _TP_CTX
        C = tp.C
        B, Tl, K = x.shape
        T, N = Tl * tp.world, weight.shape[0]
        M = B * T
        x2 = ops._as_bf16_2d(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        w = ops.weight_lp(weight)
        g0 = tp.buf("gather", M * K)
        ld = ops._pad_cols(N)
        out = torch.empty((M, ld), device=x.device, dtype=torch.bfloat16)
        flags = C.GEMM_BIAS if bias is not None else 0
        pre = None
        # a second linear on the same activation (SwiGLU's gate and up projections) reads the copy
        # the first one gathered
        again = g0.holds(x2)
        kw = dict(batch=B, T=T, gate=g0, gate_includes=0) if again else dict(batch=B, T=T, push=g0, push_src=x2,
                                                                              gate=g0)
        if gelu:
            pre = torch.empty((M, ld), device=x.device, dtype=torch.bfloat16)
            tp.launch(g0.t.view(M, K), False, w, False, M, N, K, pre, out, bias, None, flags | C.GEMM_GELU_DUAL, **kw)
        else:
            tp.launch(g0.t.view(M, K), False, w, False, M, N, K, out, None, bias, None, flags, **kw)
        ctx.save_for_backward(x2, weight, pre)
        ctx.dims = (B, T, Tl, M, N, K, ld)
        ctx.has_bias, ctx.gelu, ctx.x_dtype = bias is not None, gelu, x.dtype
        y = out[:, :N] if ld != N else out
        return y.view(B, T, N)

    @staticmethod
    def backward(ctx, dy):
        tp = _TP_CTX
        C = tp.C
        x2, weight, pre = ctx.saved_tensors
        B, T, Tl, M, N, K, ld = ctx.dims
        dy2 = ops._as_bf16_2d(dy)
        if ctx.gelu:
            dyc = dy2 if dy2.is_contiguous() else dy2.contiguous()
            prec = pre[:, :N] if ld != N else pre
            dy2 = C.gelu_bwd(dyc, prec if prec.is_contiguous() else prec.contiguous())
            ops._counters["launches"] += 1
        w = ops.weight_lp(weight)
        g1 = tp.buf("regather", M * K)
        slab = tp.buf("slab", M * K)
        dx2 = torch.empty((B * Tl, K), device=dy.device, dtype=torch.bfloat16)
        again = g1.holds(x2)
        if again:
            tp.launch(dy2, False, w, True, M, K, N, None, None, None, None, 0, batch=B, T=T, slab=slab, rs_out=dx2)
        else:
            tp.launch(dy2, False, w, True, M, K, N, None, None, None, None, 0, batch=B, T=T, push=g1, push_src=x2,
                      slab=slab, rs_out=dx2)
        dx = dx2.view(B, Tl, K)
        if ctx.x_dtype != torch.bfloat16:
            dx = dx.to(ctx.x_dtype)
        dw = db = None
        if ctx.needs_input_grad[1]:
            if not again:
                tp.wait_arrivals(g1)
            dw = ops._wgrad(C, dy2, g1.t.view(M, K), weight, N, K, M)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops._bias_grad(C, dy2, N)
        return dx, dw, db, None


class _LinearReduceScatterFn(torch.autograd.Function):
    """y[B, T/tp, N] = reduce_scatter_T(x[B, T, K/tp] W^T) + bias + residual, one launch per rank.

    Backward: one launch computes dX = all_gather_T(dY) W; the weight gradient reads the gathered dY
    that launch left in this rank's workspace."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        tp = _TP_CTX
        B, T, K = x.shape
        Tl, N = T // tp.world, weight.shape[0]
        M = B * T
        x2 = ops._as_bf16_2d(x)
        w = ops.weight_lp(weight)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(B * Tl, N)
            if res2.dtype != torch.bfloat16 or res2.stride(-1) != 1 or res2.stride(0) % 8 or res2.data_ptr() % 16:
                res2 = res2.to(torch.bfloat16).contiguous()
        out = torch.empty((B * Tl, N), device=x.device, dtype=torch.bfloat16)
        slab = tp.buf("slab", M * N)
        tp.launch(x2, False, w, False, M, N, K, None, None, None, None, 0, batch=B, T=T, slab=slab, rs_out=out,
                  rs_bias=bias, rs_residual=res2)
        ctx.save_for_backward(x2, weight)
        ctx.dims = (B, T, Tl, M, N, K)
        ctx.has_bias, ctx.has_res, ctx.x_dtype = bias is not None, residual is not None, x.dtype
        ctx.res_dtype = residual.dtype if residual is not None else None
        return out.view(B, Tl, N)

    @staticmethod
    def backward(ctx, dy):
        tp = _TP_CTX
        C = tp.C
        x2, weight = ctx.saved_tensors
        B, T, Tl, M, N, K = ctx.dims
        dy2 = ops._as_bf16_2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        w = ops.weight_lp(weight)
        g0 = tp.buf("gather", M * N)
        dx2 = torch.empty((M, K), device=dy.device, dtype=torch.bfloat16)
        tp.launch(g0.t.view(M, N), False, w, True, M, K, N, dx2, None, None, None, 0, batch=B, T=T, push=g0,
                  push_src=dy2, gate=g0)
        dx = dx2.view(B, T, K)
        if ctx.x_dtype != torch.bfloat16:
            dx = dx.to(ctx.x_dtype)
        dw = db = dres = None
        if ctx.needs_input_grad[1]:
            dw = ops._wgrad(C, g0.t.view(M, N), x2, weight, N, K, M)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops._bias_grad(C, dy2, N)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy if dy.dtype == ctx.res_dtype else dy.to(ctx.res_dtype)
        return dx, dw, db, dres


class VocabCEMerge:
    """Cross-rank merge of the vocab-parallel cross-entropy statistics in one NVLink kernel."""

    _by_ctx: Dict[int, "VocabCEMerge"] = {}

    @classmethod
    def get(cls, device: torch.device) -> Optional["VocabCEMerge"]:
        tp = _tp_context(device)
        if tp is None:
            return None
        if id(tp) not in cls._by_ctx:
            cls._by_ctx[id(tp)] = cls(tp.nvl)
        return cls._by_ctx[id(tp)]

    def __init__(self, nvl: NvlinkContext):
        self.nvl = nvl
        self.rows_cap = 0
        self.buf = None
        self.ch0 = nvl.reserve_channels(nvl.C.MAX_COMM_BLOCKS)

    def __call__(self, lse_local, row_loss, t_local, vocab_valid):
        nvl = self.nvl
        rows = lse_local.numel()
        if rows > self.rows_cap:
            self.rows_cap = max(rows, 4096)
            self.buf = nvl.alloc(2 * nvl.world * self.rows_cap, torch.float32)     # float2 [world][rows_cap]
            self.ptrs, _ = nvl.ptrs(self.buf)
        lse = torch.empty_like(lse_local)
        loss = torch.empty_like(lse_local)
        nvl.C.nvl_ce_merge(self.ptrs, nvl.flag_ptrs, lse_local.contiguous(), row_loss.contiguous(),
                           t_local.contiguous(), vocab_valid, lse, loss, self.rows_cap, nvl.rank, nvl.world, self.ch0,
                           nvl.err, nvl.epoch_ctr)
        ops._counters["launches"] += 1
        return lse, loss


class _LinearAllReduceFn(torch.autograd.Function):
    """y[B, T, N] = all_reduce(x[B, T, K/tp] W^T) + bias (+ residual) for tensor parallelism without
    sequence parallelism: the GEMM's partial rows go to their owner rank, which sums them and writes
    the result to every rank -- one launch.  Backward needs no communication."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        tp = _TP_CTX
        B, T, K = x.shape
        N = weight.shape[0]
        M = B * T
        x2 = ops._as_bf16_2d(x)
        w = ops.weight_lp(weight)
        slab = tp.buf("slab", M * N)
        full = tp.buf("allreduce", M * N)
        tp.launch(x2, False, w, False, M, N, K, None, None, None, None, 0, batch=B, T=T, slab=slab, rs_bias=bias,
                  bcast=full)
        tp.wait_arrivals(full)
        # leave the workspace at once: the next launch of the group writes into it again
        y = full.t.view(M, N)
        y = y.clone() if residual is None else y + residual.reshape(M, N).to(torch.bfloat16)
        ctx.save_for_backward(x2, weight)
        ctx.dims = (B, T, M, N, K)
        ctx.has_bias, ctx.has_res, ctx.x_dtype = bias is not None, residual is not None, x.dtype
        ctx.res_dtype = residual.dtype if residual is not None else None
        return y.view(B, T, N)

    @staticmethod
    def backward(ctx, dy):
        C = _TP_CTX.C
        x2, weight = ctx.saved_tensors
        B, T, M, N, K = ctx.dims
        dy2 = ops._as_bf16_2d(dy)
        dx = dw = db = dres = None
        if ctx.needs_input_grad[0]:
            dx2 = torch.empty((M, K), device=dy.device, dtype=torch.bfloat16)
            C.gemm(dy2, False, ops.weight_lp(weight), True, M, K, N, dx2, None, None, None, None, 0, 0)
            ops._counters["launches"] += 1
            dx = dx2.view(B, T, K)
            if ctx.x_dtype != torch.bfloat16:
                dx = dx.to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = ops._wgrad(C, dy2, x2, weight, N, K, M)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops._bias_grad(C, dy2, N)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy if dy.dtype == ctx.res_dtype else dy.to(ctx.res_dtype)
        return dx, dw, db, dres


class _CopyLinearFn(torch.autograd.Function):
    """Column-parallel linear on an input every rank holds in full (no sequence parallelism):
    y = x W^T + b needs no communication forward; backward computes dX = all_reduce(dY W) as one
    GEMM + all-reduce launch."""

    @staticmethod
    def forward(ctx, x, weight, bias, gelu):
        C = _TP_CTX.C
        B, T, K = x.shape
        N = weight.shape[0]
        M = B * T
        x2 = ops._as_bf16_2d(x)
        w = ops.weight_lp(weight)
        ld = ops._pad_cols(N)
        out = torch.empty((M, ld), device=x.device, dtype=torch.bfloat16)
        flags = C.GEMM_BIAS if bias is not None else 0
        pre = None
        if gelu:
            pre = torch.empty((M, ld), device=x.device, dtype=torch.bfloat16)
            C.gemm(x2, False, w, False, M, N, K, pre, out, bias, None, None, flags | C.GEMM_GELU_DUAL, 0)
        else:
            C.gemm(x2, False, w, False, M, N, K, out, None, bias, None, None, flags, 0)
        ops._counters["launches"] += 1
        ctx.save_for_backward(x2, weight, pre)
        ctx.dims = (B, T, M, N, K, ld)
        ctx.has_bias, ctx.gelu, ctx.x_dtype = bias is not None, gelu, x.dtype
        y = out[:, :N] if ld != N else out
        return y.view(B, T, N)

    @staticmethod
    def backward(ctx, dy):
        tp = _TP_CTX
        C = tp.C
        x2, weight, pre = ctx.saved_tensors
        B, T, M, N, K, ld = ctx.dims
        dy2 = ops._as_bf16_2d(dy)
        if ctx.gelu:
            dyc = dy2 if dy2.is_contiguous() else dy2.contiguous()
            prec = pre[:, :N] if ld != N else pre
            dy2 = C.gelu_bwd(dyc, prec if prec.is_contiguous() else prec.contiguous())
            ops._counters["launches"] += 1
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            slab = tp.buf("slab", M * K)
            full = tp.buf("allreduce", M * K)
            tp.launch(dy2, False, ops.weight_lp(weight), True, M, K, N, None, None, None, None, 0, batch=B, T=T,
                      slab=slab, bcast=full)
            tp.wait_arrivals(full)
            dx = full.t.view(B, T, K).clone()
            if ctx.x_dtype != torch.bfloat16:
                dx = dx.to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = ops._wgrad(C, dy2, x2, weight, N, K, M)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops._bias_grad(C, dy2, N)
        return dx, dw, db, None


def linear_all_reduce(x, weight, bias, residual):
    if _TP_CTX is None:
        raise RuntimeError("fused tensor-parallel kernels are not initialised")
    return _LinearAllReduceFn.apply(x, weight, bias, residual)


def copy_linear(x, weight, bias, gelu=False):
    if _TP_CTX is None:
        raise RuntimeError("fused tensor-parallel kernels are not initialised")
    return _CopyLinearFn.apply(x, weight, bias, gelu)


def allgather_linear(x, weight, bias, gelu=False):
    if _TP_CTX is None:
        raise RuntimeError("fused tensor-parallel kernels are not initialised")
    return _AllGatherLinearFn.apply(x, weight, bias, gelu)


def linear_reduce_scatter(x, weight, bias, residual):
    if _TP_CTX is None:
        raise RuntimeError("fused tensor-parallel kernels are not initialised")
    return _LinearReduceScatterFn.apply(x, weight, bias, residual)
