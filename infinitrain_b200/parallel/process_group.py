"""Process groups, asynchronous ``Work`` handles and the group factory.

Reference: infini_train/include/nn/parallel/process_group.h:40-139, infini_train/src/nn/parallel/
process_group.cc:37-454, work.cc:21-141.  The reference wraps NCCL communicators behind a ``CclImpl``
abstraction with one high-priority stream per (group, device) and a file-based unique-id
rendezvous.  Here one process drives one GPU and ``torch.distributed`` is the plumbing: NCCL over
NVLink/NVSwitch on GPUs, gloo on CPU ranks (used by the tests); the rendezvous is torch's TCP store
(``MASTER_ADDR``/``MASTER_PORT``).  The fused compute+collective kernels of
:mod:`infinitrain_b200.parallel.symm` bypass these calls and move data from inside the kernels.

Stream semantics of the five asynchronous collectives follow the reference: the call is ordered
after the work already queued on the current (compute) stream, runs on the backend's own stream,
and either returns a ``Work`` (``async_op=True``) or makes the compute stream wait for it.
"""
from __future__ import annotations

import os

import enum
import time
from datetime import timedelta
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import global_env as genv


class ReduceOpType(enum.IntEnum):
    kSum = 0
    kProd = 1
    kMin = 2
    kMax = 3
    kAvg = 4


def _to_dist_op(op: ReduceOpType, backend: str):
    if op == ReduceOpType.kAvg:
        # gloo has no AVG: the caller divides after a SUM.
        return dist.ReduceOp.AVG if backend == "nccl" else dist.ReduceOp.SUM
    return {ReduceOpType.kSum: dist.ReduceOp.SUM, ReduceOpType.kProd: dist.ReduceOp.PRODUCT,
            ReduceOpType.kMin: dist.ReduceOp.MIN, ReduceOpType.kMax: dist.ReduceOp.MAX}[op]


class CclStatus(enum.IntEnum):
    kSuccess = 0
    kInProgress = 1
    kError = 2


class Work:
    """Handle of one asynchronous collective (reference: work.h:19-30, work.cc)."""

    def __init__(self, handle=None, post=None, device: Optional[torch.device] = None, group: Optional["ProcessGroup"] = None):
        self._handle = handle
        self._group = group          # asked for the communicator's asynchronous error state
        self._post = post            # runs once after completion (e.g. the division of a gloo "avg")
        self._done = handle is None
        self._exception: Optional[BaseException] = None
        self._device = device

    def _finish(self):
        if not self._done:
            self._done = True
            if self._post is not None:
                self._post()
                self._post = None

    def WaitBlocking(self, timeout_s: float = 0.0) -> bool:
        """Blocks the host until the collective has completed.  Returns False on time-out or
        error (the exception is kept and can be read with ``exception()``)."""
        if self._done:
            return True
        try:
            if timeout_s and timeout_s > 0:
                deadline = time.monotonic() + timeout_s
                while not self._handle.is_completed():
                    if time.monotonic() > deadline:
                        return False
                    time.sleep(50e-6)
            self._handle.wait()
            if self._device is not None and self._device.type == "cuda":
                torch.cuda.current_stream(self._device).synchronize()
            self._finish()
            return True
        except Exception as e:  # noqa: BLE001
            self._exception = e
            return False

    def WaitNonBlocking(self) -> bool:
        """Makes the current stream wait for the collective; the host does not block (NCCL).  On
        CPU backends this is a blocking wait."""
        if self._done:
            return True
        try:
            self._handle.wait()
            self._finish()
            return True
        except Exception as e:  # noqa: BLE001
            self._exception = e
            return False

    Synchronize = WaitBlocking

    def IsCompleted(self) -> bool:
        if self._done:
            return True
        try:
            return bool(self._handle.is_completed())
        except Exception as e:  # noqa: BLE001
            self._exception = e
            return True

    def IsSuccess(self) -> bool:
        return self._exception is None and self.IsCompleted()

    def CheckCclStatus(self) -> CclStatus:
        """Error state of this operation and of its communicator (reference: work.cc:118-132 asks
        ``ncclCommGetAsyncError``; here the NCCL backend's watchdog keeps that state and
        ``get_error()`` reports it).  An error found this way is kept as the Work's exception."""
        if self._exception is None and self._handle is not None and hasattr(self._handle, "exception"):
            try:
                e = self._handle.exception()
                if e is not None:
                    self._exception = e if isinstance(e, BaseException) else RuntimeError(f"collective failed: {e}")
            except Exception as e:  # noqa: BLE001
                self._exception = e
        if self._exception is None and self._group is not None:
            code = self._group.AsyncError()
            if code != 0:
                self._exception = RuntimeError(f"CCL async error on group {self._group.name}: code {code}")
        if self._exception is not None:
            return CclStatus.kError
        return CclStatus.kSuccess if self.IsCompleted() else CclStatus.kInProgress

    def exception(self):
        return self._exception


class ProcessGroup:
    def __init__(self, name: str, ranks: Sequence[int], pg: Optional[dist.ProcessGroup]):
        self.name = name
        self.ranks = list(ranks)
        self.pg = pg
        self.world_size = len(self.ranks)
        self._g2l = {r: i for i, r in enumerate(self.ranks)}

    # ------------------------------------------------------------------ queries
    def GetGroupRank(self, global_rank: int) -> int:
        return self._g2l[global_rank]

    def GetGlobalRank(self, group_rank: int) -> int:
        return self.ranks[group_rank]

    def MyGroupRank(self) -> int:
        return self._g2l[genv.MyRank()]

    @property
    def backend(self) -> str:
        if self.pg is None:
            return "none"
        return dist.get_backend(self.pg)

    def _trivial(self) -> bool:
        return self.world_size <= 1 or self.pg is None

    def AsyncError(self) -> int:
        """0 = healthy.  For NCCL groups: the communicator's asynchronous error as the backend's
        watchdog sees it (1 time-out, 2 communicator error, 3 error on a remote rank)."""
        if self.pg is None:
            return 0
        try:
            backend = self.pg._get_backend(torch.device("cuda")) if self.backend == "nccl" else None
        except Exception:  # noqa: BLE001
            backend = None
        if backend is None or not hasattr(backend, "get_error"):
            return 0
        err = backend.get_error()
        return int(getattr(err, "value", err))

    def _wrap(self, handle, async_op, post=None, device=None):
        w = Work(handle, post, device, self)
        if not async_op:
            w.WaitNonBlocking()
            return None
        return w

    # ------------------------------------------------------------------ collectives
    def AllReduce(self, tensor: torch.Tensor, op: ReduceOpType = ReduceOpType.kSum, async_op: bool = False):
        if self._trivial():
            return Work() if async_op else None
        backend = self.backend
        post = None
        if op == ReduceOpType.kAvg and backend != "nccl":
            n = self.world_size
            post = lambda: tensor.div_(n)  # noqa: E731
        h = dist.all_reduce(tensor, op=_to_dist_op(op, backend), group=self.pg, async_op=True)
        return self._wrap(h, async_op, post, tensor.device)

    def AllGather(self, output: torch.Tensor, input: torch.Tensor, async_op: bool = False):
        if self._trivial():
            output.copy_(input)
            return Work() if async_op else None
        inp = input.contiguous()
        if self.backend != "nccl":
            inp = inp.clone()   # only NCCL defines the in-place form (input a slice of output)
        h = dist.all_gather_into_tensor(output, inp, group=self.pg, async_op=True)
        return self._wrap(h, async_op, None, output.device)

    def ReduceScatter(self, output: torch.Tensor, input: torch.Tensor, op: ReduceOpType = ReduceOpType.kSum,
                      async_op: bool = False):
        if self._trivial():
            output.copy_(input)
            return Work() if async_op else None
        backend = self.backend
        if backend == "gloo":
            # gloo has no reduce-scatter: all-reduce a copy and keep this rank's slice.
            tmp = input.clone()
            dist.all_reduce(tmp, op=_to_dist_op(op, backend), group=self.pg)
            if op == ReduceOpType.kAvg:
                tmp.div_(self.world_size)
            r = self.MyGroupRank()
            output.copy_(tmp.view(self.world_size, -1)[r].view_as(output))
            return Work() if async_op else None
        h = dist.reduce_scatter_tensor(output, input.contiguous(), op=_to_dist_op(op, backend), group=self.pg,
                                       async_op=True)
        return self._wrap(h, async_op, None, output.device)

    def BroadCast(self, tensor: torch.Tensor, src_group_rank: int = 0, async_op: bool = False):
        if self._trivial():
            return Work() if async_op else None
        h = dist.broadcast(tensor, src=self.ranks[src_group_rank], group=self.pg, async_op=True)
        return self._wrap(h, async_op, None, tensor.device)

    def Reduce(self, tensor: torch.Tensor, dst_group_rank: int = 0, op: ReduceOpType = ReduceOpType.kSum,
               async_op: bool = False):
        if self._trivial():
            return Work() if async_op else None
        h = dist.reduce(tensor, dst=self.ranks[dst_group_rank], op=_to_dist_op(op, self.backend), group=self.pg,
                        async_op=True)
        return self._wrap(h, async_op, None, tensor.device)

    def Send(self, tensors: Sequence[torch.Tensor], dst_group_rank: int, async_op: bool = False):
        works = [dist.isend(t.contiguous(), dst=self.ranks[dst_group_rank], group=self.pg) for t in tensors]
        return self._p2p(works, async_op)

    def Recv(self, tensors: Sequence[torch.Tensor], src_group_rank: int, async_op: bool = False):
        works = [dist.irecv(t, src=self.ranks[src_group_rank], group=self.pg) for t in tensors]
        return self._p2p(works, async_op)

    def BatchSendRecv(self, ops: Sequence[tuple], async_op: bool = False):
        """``ops`` is a list of (is_send, tensor, peer group rank).  All transfers progress together
        (one NCCL group), so two ranks that each send to and receive from the other in one exchange
        cannot block one another; transfers between one pair of ranks match in list order."""
        if not ops:
            return None
        p2p = [dist.P2POp(dist.isend if is_send else dist.irecv, t, self.ranks[peer], group=self.pg)
               for is_send, t, peer in ops]
        return self._p2p(dist.batch_isend_irecv(p2p), async_op)

    def _p2p(self, works, async_op):
        class _Multi:
            def __init__(self, ws):
                self.ws = ws

            def wait(self):
                for w in self.ws:
                    w.wait()

            def is_completed(self):
                return all(w.is_completed() for w in self.ws)

        w = Work(_Multi(works), group=self)
        if not async_op:
            w.WaitNonBlocking()
            return None
        return w

    def Barrier(self):
        if not self._trivial():
            dist.barrier(group=self.pg)

    def abort(self) -> bool:
        """Tears the communicator down without waiting for outstanding collectives (``ncclCommAbort``
        for NCCL; backends without an abort return False).  Used by the failure watchdog."""
        if self._trivial():
            return False
        fn = getattr(dist.distributed_c10d, "_abort_process_group", None)
        if fn is None or self.backend != "nccl":
            return False
        try:
            fn(self.pg)
            return True
        except Exception:  # noqa: BLE001
            return False

    # ------------------------------------------------------------------ legacy data-parallel helpers
    def ReduceAddCoalesced(self, tensors: Sequence[torch.Tensor], dst_group_rank: int = 0):
        """Sum every tensor of the list onto ``dst`` (reference: process_group.cc:292-330)."""
        for t in tensors:
            self.Reduce(t, dst_group_rank, ReduceOpType.kSum)
        return list(tensors)

    def Scatter(self, tensor: Optional[torch.Tensor], out: torch.Tensor, src_group_rank: int = 0, dim: int = 0):
        if self._trivial():
            out.copy_(tensor)
            return out
        chunks = None
        if self.MyGroupRank() == src_group_rank:
            chunks = [c.contiguous() for c in tensor.chunk(self.world_size, dim)]
        dist.scatter(out, chunks, src=self.ranks[src_group_rank], group=self.pg)
        return out

    def Gather(self, tensor: torch.Tensor, dst_group_rank: int = 0, dim: int = 0):
        if self._trivial():
            return tensor
        outs = None
        if self.MyGroupRank() == dst_group_rank:
            outs = [torch.empty_like(tensor) for _ in range(self.world_size)]
        dist.gather(tensor.contiguous(), outs, dst=self.ranks[dst_group_rank], group=self.pg)
        return torch.cat(outs, dim) if outs is not None else None


class ProcessGroupFactory:
    """Creates and caches the named groups: ``default`` and ``DP<i>`` / ``TP<i>`` / ``PP<i>``.

    ``torch.distributed.new_group`` is collective over the whole world, so every group of every axis
    is created by every process in one fixed order at ``Init`` (the reference creates them lazily
    per thread with a condition variable, process_group.h:123-139).
    """

    kDefaultProcessGroupName = "default"
    _instance: Optional["ProcessGroupFactory"] = None

    def __init__(self):
        self.groups: Dict[str, ProcessGroup] = {}
        self.initialized = False

    @classmethod
    def Instance(cls, device_type=None) -> "ProcessGroupFactory":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    @classmethod
    def Reset(cls):
        cls._instance = None

    def Init(self, backend: Optional[str] = None, timeout_s: float = 600.0, device: Optional[torch.device] = None,
             rendezvous_file: Optional[str] = None):
        """Creates the job's groups.  Rendezvous is a TCP store (``MASTER_ADDR`` / ``MASTER_PORT``) or,
        when ``rendezvous_file`` / ``ITB_RDZV_FILE`` names a path on a filesystem all ranks share, a
        file there (the reference's only scheme: src/core/ccl/ccl_utils.cc:14-53); the file must not
        exist before the job starts."""
        if self.initialized:
            return self
        world = genv.GetWorldSize()
        rank = genv.MyRank()
        if os.environ.get("ITB_PG_TIMEOUT_S"):   # rendezvous and collective time-out of this job, in seconds
            timeout_s = float(os.environ["ITB_PG_TIMEOUT_S"])
        if world > 1 and not dist.is_initialized():
            if backend is None:
                backend = "nccl" if (device is not None and device.type == "cuda") else "gloo"
            kwargs = {}
            if backend == "nccl" and device is not None:
                kwargs["device_id"] = device
            rendezvous_file = rendezvous_file or os.environ.get("ITB_RDZV_FILE")
            if rendezvous_file:
                kwargs["init_method"] = "file://" + os.path.abspath(rendezvous_file)
            dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                    timeout=timedelta(seconds=timeout_s), **kwargs)
        if world <= 1 or not dist.is_initialized():
            self.groups[self.kDefaultProcessGroupName] = ProcessGroup(self.kDefaultProcessGroupName, [0], None)
            for ax in genv.Axis:
                self.groups[f"{ax.name}0"] = ProcessGroup(f"{ax.name}0", [0], None)
            self.initialized = True
            return self
        self.groups[self.kDefaultProcessGroupName] = ProcessGroup(self.kDefaultProcessGroupName, list(range(world)),
                                                                  dist.group.WORLD)
        L = genv.GlobalEnv.Instance().layout
        for ax in genv.Axis:
            seen = {}
            for r in range(world):
                gid = L.GroupId(ax, *L.CoordOf(r))
                if gid not in seen:
                    seen[gid] = L.GroupRanks(ax, *L.CoordOf(r))
            for gid in sorted(seen):
                ranks = seen[gid]
                name = f"{ax.name}{gid}"
                pg = dist.new_group(ranks=ranks, timeout=timedelta(seconds=timeout_s)) if len(ranks) > 1 else None
                if rank in ranks:
                    self.groups[name] = ProcessGroup(name, ranks, pg)
        self.initialized = True
        return self

    def GetOrCreate(self, name: str, ranks: Optional[Sequence[int]] = None) -> ProcessGroup:
        if name in self.groups:
            return self.groups[name]
        if ranks is None:
            raise KeyError(f"process group '{name}' does not exist")
        pg = dist.new_group(ranks=list(ranks)) if (len(ranks) > 1 and dist.is_initialized()) else None
        self.groups[name] = ProcessGroup(name, ranks, pg)
        return self.groups[name]

    def Get(self, name: str) -> ProcessGroup:
        return self.groups[name]

    def GetDefaultProcessGroup(self) -> ProcessGroup:
        return self.groups[self.kDefaultProcessGroupName]

    # convenience: the groups of the calling rank
    def dp_group(self) -> ProcessGroup:
        return self.groups[genv.GetDataParallelProcessGroupName(genv.MyRank())]

    def tp_group(self) -> ProcessGroup:
        return self.groups[genv.GetTensorParallelProcessGroupName(genv.MyRank())]

    def pp_group(self) -> ProcessGroup:
        return self.groups[genv.GetPipelineParallelProcessGroupName(genv.MyRank())]


def tp_group() -> Optional[ProcessGroup]:
    f = ProcessGroupFactory.Instance()
    return f.tp_group() if f.initialized else None


def dp_group() -> Optional[ProcessGroup]:
    f = ProcessGroupFactory.Instance()
    return f.dp_group() if f.initialized else None


def pp_group() -> Optional[ProcessGroup]:
    f = ProcessGroupFactory.Instance()
    return f.pp_group() if f.initialized else None
