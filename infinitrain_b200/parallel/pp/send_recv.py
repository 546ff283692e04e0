"""Point-to-point transfers between pipeline stages.

Reference: infini_train/src/nn/parallel/pp/send_recv.cc:58-109 — ``ISend`` / ``IRecv`` are autograd
functions whose backward is the opposite transfer (the gradient of a sent activation is received
from the consumer, the gradient of a received activation is sent back to the producer).  The
payload keeps the activation dtype (bf16 under autocast); the reference hard-codes fp32.
Transfers stay on NCCL point-to-point (gloo on CPU ranks).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..process_group import ProcessGroup, pp_group


class _ISendFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pg, peer):
        ctx.pg, ctx.peer, ctx.meta = pg, peer, (x.shape, x.dtype, x.device)
        pg.Send([x.detach().contiguous()], peer, async_op=False)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, _dummy):
        shape, dtype, device = ctx.meta
        g = torch.empty(shape, dtype=dtype, device=device)
        ctx.pg.Recv([g], ctx.peer, async_op=False)
        return g, None, None


class _IRecvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf, pg, peer):
        ctx.pg, ctx.peer = pg, peer
        pg.Recv([buf], peer, async_op=False)
        return buf.view_as(buf)

    @staticmethod
    def backward(ctx, g):
        ctx.pg.Send([g.contiguous()], ctx.peer, async_op=False)
        return None, None, None


def ISend(tensors: Sequence[torch.Tensor], peer_stage: int, pg: Optional[ProcessGroup] = None) -> List[torch.Tensor]:
    """Sends every tensor to ``peer_stage``; the returned tensors carry a grad_fn whose backward
    RECEIVES the gradient from that stage."""
    pg = pg or pp_group()
    return [_ISendFn.apply(t, pg, peer_stage) for t in tensors]


def IRecv(buffers: Sequence[torch.Tensor], peer_stage: int, pg: Optional[ProcessGroup] = None) -> List[torch.Tensor]:
    """Receives into ``buffers`` (which must require grad) from ``peer_stage``; backward SENDS the
    gradient back."""
    pg = pg or pp_group()
    return [_IRecvFn.apply(b, pg, peer_stage) for b in buffers]
