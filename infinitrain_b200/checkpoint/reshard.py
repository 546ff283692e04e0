"""Elastic resume: re-shard ZeRO optimizer state saved by ``old_dp`` data-parallel ranks for a run
with ``new_dp`` ranks.

``DistributedOptimizer`` keeps one state tensor per bucket and rank (``adam.m.<bucket>``,
``adam.v.<bucket>``: that rank's 1/dp slice of the bucket), and the flat layout -- parameter offsets,
bucket boundaries, end padding to ``lcm(dp, 128)`` -- is a pure function of the parameter sizes and of
``dp`` (:func:`plan_flat_layout`).  So the state of any other ``dp`` follows from the per-rank files
without the model: stitch the old shards into the old flat buffer, move every parameter's span to
its place in the new flat buffer, cut the new rank's slices.  The reference refuses to resume on a
different topology (checkpoint_manager.cc:56-63).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Sequence

import torch

from ..parallel.ddp.param_and_grad_buffer import plan_flat_layout


def reshard_zero_optimizer_state(old_states: Sequence[Dict[str, torch.Tensor]], numels: Sequence[int], new_dp: int,
                                 new_rank: int, bucket_size_in_elements: int = 1_000_000,
                                 pad_for_busbw: bool = False, first_bucket_index: int = 0,
                                 keys: Sequence[str] = ("adam.m", "adam.v")) -> "OrderedDict[str, torch.Tensor]":
    """``old_states[r]`` is rank r's optimizer state dict; ``numels`` are the element counts of the
    parameters of one flat buffer in registration order.  Returns the state dict of ``new_rank`` in a
    run with ``new_dp`` ranks.  Scalar entries (``adam.t``) are copied from rank 0."""
    old_dp = len(old_states)
    if not (0 <= new_rank < new_dp):
        raise ValueError("new_rank out of range")
    old = plan_flat_layout(list(numels), old_dp, shard=True, bucket_size_in_elements=bucket_size_in_elements,
                           pad_for_busbw=pad_for_busbw)
    new = plan_flat_layout(list(numels), new_dp, shard=True, bucket_size_in_elements=bucket_size_in_elements,
                           pad_for_busbw=pad_for_busbw)
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    for key in keys:
        flat_old = None
        for b, (bs, be) in enumerate(old.bucket_ranges):
            n = (be - bs) // old_dp
            for r in range(old_dp):
                name = f"{key}.{first_bucket_index + b}"
                if name not in old_states[r]:
                    raise KeyError(f"rank {r} has no optimizer state {name}")
                piece = old_states[r][name].reshape(-1)
                if piece.numel() != n:
                    raise ValueError(f"{name} of rank {r} has {piece.numel()} elements, the layout says {n}")
                if flat_old is None:
                    flat_old = torch.zeros(old.numel, dtype=piece.dtype)
                flat_old[bs + r * n: bs + (r + 1) * n] = piece.cpu()
        flat_new = torch.zeros(new.numel, dtype=flat_old.dtype)
        for (s0, e0, _), (s1, e1, _) in zip(old.param_ranges, new.param_ranges):
            flat_new[s1:e1] = flat_old[s0:e0]
        for b, (bs, be) in enumerate(new.bucket_ranges):
            n = (be - bs) // new_dp
            out[f"{key}.{first_bucket_index + b}"] = flat_new[bs + new_rank * n: bs + (new_rank + 1) * n].clone()
    for name, value in old_states[0].items():
        if not any(name.startswith(k + ".") for k in keys):
            out[name] = value.clone() if isinstance(value, torch.Tensor) else value
    return out


def gather_full_optimizer_state(old_states: Sequence[Dict[str, torch.Tensor]], numels: Sequence[int],
                                **kw) -> List[Dict[str, torch.Tensor]]:
    """Per-parameter state (``[{"adam.m": tensor, "adam.v": tensor}, ...]`` in parameter order) from
    the sharded files: the ``new_dp == 1`` re-shard cut at the parameter boundaries."""
    one = reshard_zero_optimizer_state(old_states, numels, 1, 0, **kw)
    layout = plan_flat_layout(list(numels), 1, shard=True,
                              bucket_size_in_elements=kw.get("bucket_size_in_elements", 1_000_000),
                              pad_for_busbw=kw.get("pad_for_busbw", False))
    keys = kw.get("keys", ("adam.m", "adam.v"))
    first = kw.get("first_bucket_index", 0)
    res = []
    for (s, e, b) in layout.param_ranges:
        bs, _ = layout.bucket_ranges[b]
        res.append({k: one[f"{k}.{first + b}"][s - bs: e - bs].clone() for k in keys})
    return res
