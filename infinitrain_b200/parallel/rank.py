"""Rank coordinates (reference: infini_train/src/nn/parallel/rank.cc:14)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Rank:
    process_rank: int = 0
    thread_rank: int = 0
    process_size: int = 1
    thread_size: int = 1

    def GlobalRank(self) -> int:
        return self.process_rank * self.thread_size + self.thread_rank

    def WorldSize(self) -> int:
        return self.process_size * self.thread_size

    def IsParallel(self) -> bool:
        return self.WorldSize() > 1

    def IsMainRank(self) -> bool:
        return self.GlobalRank() == 0

    def IsLastRank(self) -> bool:
        return self.GlobalRank() == self.WorldSize() - 1
