"""Global parallel environment and the 3-axis rank layout.

Reference: infini_train/include/nn/parallel/global.h:17-155, infini_train/src/nn/parallel/global.cc.
The process model differs on purpose: one PROCESS per GPU (the reference runs one thread per GPU
inside a process), so "threads per process" is accepted and treated as local ranks.  Environment
variables: the reference's launcher names (NNODES, NPROC_PER_NODE, PROC_WORLD_SIZE,
GLOBAL_PROC_RANK, LOCAL_PROC_RANK) and torchrun's (WORLD_SIZE, RANK, LOCAL_RANK) are both read.

Layout: data-, tensor- and pipeline-parallel axes with TP fastest, then DP, then PP, so a TP group
sits on adjacent GPUs: ``rank = tp + TP * dp + TP * DP * pp``.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, field
from typing import List, Tuple


class Axis(enum.IntEnum):
    DP = 0
    TP = 1
    PP = 2


AXIS_COUNT = 3


@dataclass
class Layout:
    sizes: List[int] = field(default_factory=lambda: [1, 1, 1])       # indexed by Axis
    order: Tuple[Axis, ...] = (Axis.TP, Axis.DP, Axis.PP)             # fastest-varying first
    strides: List[int] = field(default_factory=lambda: [1, 1, 1])

    def InitStrides(self) -> None:
        stride = 1
        for ax in self.order:
            self.strides[ax] = stride
            stride *= self.sizes[ax]

    def RankOf(self, dp: int, tp: int, pp: int) -> int:
        coord = (dp, tp, pp)
        return sum(coord[ax] * self.strides[ax] for ax in Axis)

    def CoordOf(self, rank: int) -> Tuple[int, int, int]:
        return tuple((rank // self.strides[ax]) % self.sizes[ax] for ax in Axis)  # (dp, tp, pp)

    def GroupId(self, target: Axis, dp: int, tp: int, pp: int) -> int:
        coord = (dp, tp, pp)
        gid, mult = 0, 1
        for ax in reversed(self.order):
            if ax == target:
                continue
            gid += coord[ax] * mult
            mult *= self.sizes[ax]
        return gid

    def GroupRanks(self, target: Axis, dp: int, tp: int, pp: int) -> List[int]:
        coord = [dp, tp, pp]
        out = []
        for v in range(self.sizes[target]):
            coord[target] = v
            out.append(self.RankOf(*coord))
        return out

    def NumGroups(self, target: Axis) -> int:
        n = 1
        for ax in Axis:
            if ax != target:
                n *= self.sizes[ax]
        return n


def _env_int(names, default):
    for n in names:
        v = os.environ.get(n)
        if v not in (None, ""):
            return int(v)
    return default


class GlobalEnv:
    _instance = None

    def __init__(self):
        self.initialized = False
        self.nnodes = 1
        self.nproc_per_node = 1
        self.nthread_per_process = 1
        self.world_size = 1
        self.global_proc_rank = 0
        self.local_proc_rank = 0
        self.tensor_parallel_size = 1
        self.sequence_parallel_enabled = False
        self.data_parallel_size = 1
        self.pipeline_parallel_size = 1
        self.virtual_pipeline_parallel_size = 1
        self.layout = Layout()

    @classmethod
    def Instance(cls) -> "GlobalEnv":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def Init(self, nthread_per_process: int = 1, tensor_parallel_size: int = 1,
             sequence_parallel_enabled: bool = False, pipeline_parallel_size: int = 1,
             virtual_pipeline_parallel_size: int = 1, world_size: int | None = None,
             rank: int | None = None) -> None:
        self.nnodes = _env_int(["NNODES"], 1)
        world_env = _env_int(["WORLD_SIZE", "PROC_WORLD_SIZE"], 1)
        self.nproc_per_node = _env_int(["NPROC_PER_NODE", "LOCAL_WORLD_SIZE"], max(1, world_env // self.nnodes))
        self.nthread_per_process = nthread_per_process
        self.world_size = world_size if world_size is not None else max(world_env, 1)
        self.global_proc_rank = rank if rank is not None else _env_int(["RANK", "GLOBAL_PROC_RANK"], 0)
        self.local_proc_rank = _env_int(["LOCAL_RANK", "LOCAL_PROC_RANK"], self.global_proc_rank % max(1, self.nproc_per_node))
        tp, pp = tensor_parallel_size, pipeline_parallel_size
        if self.world_size % (tp * pp) != 0:
            raise ValueError(f"world size {self.world_size} is not divisible by tp*pp = {tp * pp}")
        if sequence_parallel_enabled and tp <= 1:
            sequence_parallel_enabled = False
        self.tensor_parallel_size = tp
        self.sequence_parallel_enabled = sequence_parallel_enabled
        self.pipeline_parallel_size = pp
        self.virtual_pipeline_parallel_size = virtual_pipeline_parallel_size
        self.data_parallel_size = self.world_size // (tp * pp)
        self.layout = Layout()
        self.layout.sizes[Axis.DP] = self.data_parallel_size
        self.layout.sizes[Axis.TP] = tp
        self.layout.sizes[Axis.PP] = pp
        self.layout.InitStrides()
        self.initialized = True

    @property
    def sequence_parallel_size(self) -> int:
        return self.tensor_parallel_size if self.sequence_parallel_enabled else 1


def InitAllEnv(nthread_per_process: int = 1, tensor_parallel_size: int = 1, sequence_parallel_enabled: bool = False,
               pipeline_parallel_size: int = 1, virtual_pipeline_parallel: int = 1, world_size=None, rank=None):
    GlobalEnv.Instance().Init(nthread_per_process, tensor_parallel_size, sequence_parallel_enabled,
                              pipeline_parallel_size, virtual_pipeline_parallel, world_size, rank)


def _g() -> GlobalEnv:
    return GlobalEnv.Instance()


def GetNnodes(): return _g().nnodes
def GetWorldSize(): return _g().world_size
def GetNprocPerNode(): return _g().nproc_per_node
def GetNthreadPerProc(): return _g().nthread_per_process
def GetGlobalProcRank(): return _g().global_proc_rank
def GetLocalProcRank(): return _g().local_proc_rank
def GetTensorParallelSize(): return _g().tensor_parallel_size
def GetSequenceParallelSize(): return _g().sequence_parallel_size
def GetSequenceParallelEnabled(): return _g().sequence_parallel_enabled
def GetDataParallelSize(): return _g().data_parallel_size
def GetPipelineParallelSize(): return _g().pipeline_parallel_size
def GetVirtualPipelineParallelSize(): return _g().virtual_pipeline_parallel_size


def GetRankOf(dp, tp, pp): return _g().layout.RankOf(dp, tp, pp)
def GetCoordOf(rank): return _g().layout.CoordOf(rank)


def GetGroupId(target: Axis, rank: int) -> int:
    return _g().layout.GroupId(target, *GetCoordOf(rank))


def GetGroupRanks(target: Axis, rank: int) -> List[int]:
    return _g().layout.GroupRanks(target, *GetCoordOf(rank))


# Per-rank coordinates (the reference keeps these in thread-local variables).
def MyRank() -> int: return _g().global_proc_rank
def MyCoord(): return GetCoordOf(MyRank())
def GetDataParallelRank(): return MyCoord()[0]
def GetTensorParallelRank(): return MyCoord()[1]
def GetPipelineParallelRank(): return MyCoord()[2]


def GetDataParallelProcessGroupName(rank: int) -> str: return f"DP{GetGroupId(Axis.DP, rank)}"
def GetTensorParallelProcessGroupName(rank: int) -> str: return f"TP{GetGroupId(Axis.TP, rank)}"
def GetPipelineParallelProcessGroupName(rank: int) -> str: return f"PP{GetGroupId(Axis.PP, rank)}"


def ProcessGroupOverview(skip_trivial_axes: bool = True) -> str:
    """Dump of every DP / TP / PP group, in the reference's text (src/nn/parallel/global.cc:196-257):
    groups in group-id order with the coordinates that are fixed inside them."""
    L = _g().layout
    out = ["", "=== Parallel Communication Groups ===",
           f"world_size = {_g().world_size}, config: {{DP={L.sizes[Axis.DP]}, TP={L.sizes[Axis.TP]}, "
           f"PP={L.sizes[Axis.PP]}}}, order: {{" + " -> ".join(ax.name for ax in L.order) + "}"]
    axes = list(Axis)
    for k, ax in enumerate(axes):
        if skip_trivial_axes and L.sizes[ax] <= 1:
            out.append(f"[{ax.name}] size={L.sizes[ax]}, unenabled")
            continue
        groups = []
        for dp in range(1 if ax == Axis.DP else L.sizes[Axis.DP]):
            for tp in range(1 if ax == Axis.TP else L.sizes[Axis.TP]):
                for pp in range(1 if ax == Axis.PP else L.sizes[Axis.PP]):
                    groups.append((L.GroupId(ax, dp, tp, pp), (dp, tp, pp)))
        groups.sort(key=lambda g: g[0])
        out.append(f"[{ax.name}] size={L.sizes[ax]}, num_groups={L.NumGroups(ax)}")
        for gid, (dp, tp, pp) in groups:
            ranks = ", ".join(str(r) for r in sorted(L.GroupRanks(ax, dp, tp, pp)))
            c = ["-" if ax == a2 else str(v) for a2, v in zip((Axis.DP, Axis.TP, Axis.PP), (dp, tp, pp))]
            out.append(f"  - {ax.name} {gid} (dp={c[0]}, tp={c[1]}, pp={c[2]}): [{ranks}]")
        if k + 1 < len(axes):
            out.append("")
    return "\n".join(out) + "\n\n"
