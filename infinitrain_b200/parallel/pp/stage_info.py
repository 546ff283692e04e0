"""Layer-to-stage partitioning (reference: infini_train/src/nn/parallel/pp/pipeline_parallel.cc:42-77).

``total_layers`` are cut into ``pp_size * chunks_per_stage`` global chunks; the first
``total_layers % n_chunks`` chunks get one extra layer; stage ``rank`` owns the global chunks
``local * pp_size + rank`` (non-adjacent chunks: the interleaved / virtual-pipeline layout).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Tuple


@dataclass
class StageInfo:
    is_first_stage: bool
    is_last_stage: bool
    layer_ranges_per_chunk: List[Tuple[int, int]] = field(default_factory=list)


def GetStageInfo(total_layers: int, pp_size: int, rank: int, chunks_per_stage: int = 1) -> StageInfo:
    n_chunks = pp_size * chunks_per_stage
    base, rem = divmod(total_layers, n_chunks)
    ranges = []
    for local in range(chunks_per_stage):
        g = local * pp_size + rank
        if g < rem:
            start = g * (base + 1)
            end = start + base + 1
        else:
            start = rem * (base + 1) + (g - rem) * base
            end = start + base
        end = min(end, total_layers)
        if start < end:
            ranges.append((start, end))
    return StageInfo(rank == 0, rank == pp_size - 1, ranges)
