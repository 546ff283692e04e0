"""Free-function collectives and the helpers of the legacy single-process DataParallel.

Reference: infini_train/src/nn/parallel/parallel_functional.cc:16-143.
"""
from __future__ import annotations

import copy
from typing import List, Optional, Sequence

import torch

from .process_group import ProcessGroup, ProcessGroupFactory, ReduceOpType


def _pg(pg: Optional[ProcessGroup]) -> ProcessGroup:
    return pg if pg is not None else ProcessGroupFactory.Instance().GetDefaultProcessGroup()


def AllReduce(tensor, op: ReduceOpType = ReduceOpType.kSum, pg: Optional[ProcessGroup] = None, async_op: bool = False):
    return _pg(pg).AllReduce(tensor, op, async_op)


def AllGather(output, input, pg: Optional[ProcessGroup] = None, async_op: bool = False):
    return _pg(pg).AllGather(output, input, async_op)


def ReduceScatter(output, input, op: ReduceOpType = ReduceOpType.kSum, pg: Optional[ProcessGroup] = None,
                  async_op: bool = False):
    return _pg(pg).ReduceScatter(output, input, op, async_op)


def Send(tensors, dst: int, pg: Optional[ProcessGroup] = None, async_op: bool = False):
    return _pg(pg).Send(tensors, dst, async_op)


def Recv(tensors, src: int, pg: Optional[ProcessGroup] = None, async_op: bool = False):
    return _pg(pg).Recv(tensors, src, async_op)


# ---------------------------------------------------------------- single-process multi-device helpers
def Scatter(tensor: torch.Tensor, devices: Sequence[torch.device], dim: int = 0) -> List[torch.Tensor]:
    """Splits ``tensor`` into ``len(devices)`` chunks along ``dim`` and moves chunk i to device i."""
    return [c.to(d) for c, d in zip(tensor.chunk(len(devices), dim), devices)]


def Gather(tensors: Sequence[torch.Tensor], target: torch.device, dim: int = 0) -> torch.Tensor:
    return torch.cat([t.to(target) for t in tensors], dim)


def BroadcastCoalescedReshape(tensors: Sequence[torch.Tensor], devices: Sequence[torch.device]):
    """Every tensor copied to every device: result[d][i] is tensor i on device d."""
    return [[t.to(d) for t in tensors] for d in devices]


def Replicate(network: torch.nn.Module, devices: Sequence[torch.device]) -> List[torch.nn.Module]:
    """One deep copy of ``network`` per device with parameters broadcast from the original."""
    reps = []
    for d in devices:
        r = copy.deepcopy(network)
        r.to(d)
        reps.append(r)
    return reps
