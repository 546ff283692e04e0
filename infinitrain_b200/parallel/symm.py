"""Symmetric memory and the fused compute+collective kernels over NVLink / NVSwitch.

Every rank of a group allocates the same buffer through ``torch.distributed._symmetric_memory``
(CUDA VMM allocations exchanged between the processes, peer-mapped, plus an NVLS multicast mapping
when the switch supports it).  The hand-written kernels of ``csrc/comm`` then read and write peers
directly (``ld/st/red`` on peer pointers, ``multimem.ld_reduce`` / ``multimem.st`` on the multicast
pointer) and synchronise through flags in the signal pad with bounded waits.

Nothing in this module runs on CPU ranks: gloo tests exercise the NCCL/gloo formulation of the same
operations in :mod:`tensor_parallel` and :mod:`ddp`.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

_STATE: Dict[str, object] = {"tp_fused": None}


def fused_tp_enabled(x: torch.Tensor) -> bool:
    """True when the fused all-gather+GEMM / GEMM+reduce-scatter kernels should serve ``x``."""
    if not x.is_cuda:
        return False
    flag = _STATE["tp_fused"]
    if flag is None:
        flag = os.environ.get("ITB_FUSED_TP", "0") == "1"
        _STATE["tp_fused"] = flag
    return bool(flag) and _TP_CTX is not None


_TP_CTX = None


def allgather_linear(x, weight, bias, gelu=False):
    raise RuntimeError("fused tensor-parallel kernels are not initialised")


def linear_reduce_scatter(x, weight, bias, residual):
    raise RuntimeError("fused tensor-parallel kernels are not initialised")
