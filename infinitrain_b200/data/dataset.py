"""Datasets and loaders.

Reference: infini_train/include/dataset.h, infini_train/src/dataloader.cc:17-102,
example/common/tiny_shakespeare_dataset.cc:27-118.  ``DistributedDataLoader`` starts at batch
``ddp_rank`` and strides by ``ddp_world_size`` batches; there is no shuffling; in the token dataset
``y`` is ``x`` shifted by one token inside the flat token stream.  The token file is memory-mapped by
the native runtime and batches are assembled by a background thread into pinned host buffers (the
reference memcpy-stacks samples on the training thread).
"""
from __future__ import annotations

import struct
from typing import Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _ext

kGpt2TokenMagic = 20240520     # uint16 tokens
kLlama3TokenMagic = 20240801   # uint32 tokens


class Dataset:
    def __getitem__(self, idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def Size(self) -> int:
        raise NotImplementedError

    def __len__(self) -> int:
        return self.Size()


def write_token_file(path: str, tokens: Sequence[int], llama3: bool = False) -> None:
    """Writes an llm.c token file (1024-byte header: magic, version, num_tokens; then the tokens)."""
    arr = np.asarray(tokens, dtype=np.uint32 if llama3 else np.uint16)
    header = np.zeros(256, dtype=np.int32)
    header[0] = kLlama3TokenMagic if llama3 else kGpt2TokenMagic
    header[1] = 7 if llama3 else 1
    header[2] = arr.size
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(arr.tobytes())


class TinyShakespeareDataset(Dataset):
    """llm.c token file as (x, y) samples of ``sequence_length`` tokens; samples 0 .. num_seq - 2."""

    def __init__(self, filepath: str, sequence_length: int):
        self.path = filepath
        self.sequence_length = sequence_length
        self._native = None
        C = _ext.load(required=False)
        if C is not None:
            self._native = C.TokenFile(filepath)
            self.num_tokens = int(self._native.num_tokens)
            self.magic = int(self._native.magic)
        else:
            with open(filepath, "rb") as f:
                header = np.frombuffer(f.read(1024), dtype=np.int32)
                self.magic, self.num_tokens = int(header[0]), int(header[2])
                dt = np.uint16 if self.magic == kGpt2TokenMagic else np.uint32
                self._tokens = np.frombuffer(f.read(), dtype=dt)[: self.num_tokens].astype(np.int64)
        if self.magic not in (kGpt2TokenMagic, kLlama3TokenMagic):
            raise ValueError(f"unknown token file magic {self.magic}")
        max_len = 1024 if self.magic == kGpt2TokenMagic else 8192
        if sequence_length > max_len:
            raise ValueError(f"sequence length {sequence_length} exceeds the model family's limit {max_len}")
        self.num_samples = self.num_tokens // sequence_length - 1

    def Size(self) -> int:
        return self.num_samples

    def __getitem__(self, idx: int):
        T = self.sequence_length
        if self._native is not None:
            return self._native.sample(idx, T)
        s = idx * T
        return (torch.from_numpy(self._tokens[s:s + T].copy()), torch.from_numpy(self._tokens[s + 1:s + T + 1].copy()))

    def native_file(self):
        return self._native


class DataLoader:
    """Sequential batches of stacked samples (no shuffle, no workers), as in the reference."""

    def __init__(self, dataset: Dataset, batch_size: int):
        self.dataset, self.batch_size = dataset, batch_size

    def _num_batches(self) -> int:
        return self.dataset.Size() // self.batch_size

    def batch(self, b: int):
        xs, ys = zip(*(self.dataset[b * self.batch_size + i] for i in range(self.batch_size)))
        return torch.stack(xs), torch.stack(ys)

    def __iter__(self) -> Iterator:
        for b in range(self._num_batches()):
            yield self.batch(b)

    def __len__(self):
        return self._num_batches()


class DistributedDataLoader(DataLoader):
    """Rank ``ddp_rank`` reads batches ``ddp_rank, ddp_rank + W, ddp_rank + 2 W, ...``.

    For token datasets backed by the native runtime the batches come from a prefetching
    ``TokenBatcher`` (pinned host memory, ready for an asynchronous host-to-device copy).
    """

    def __init__(self, dataset: Dataset, batch_size: int, ddp_rank: int = 0, ddp_world_size: int = 1,
                 prefetch_depth: int = 4, pin_memory: Optional[bool] = None):
        super().__init__(dataset, batch_size)
        self.ddp_rank, self.ddp_world_size = ddp_rank, ddp_world_size
        self.prefetch_depth = prefetch_depth
        self.pin = torch.cuda.is_available() if pin_memory is None else pin_memory

    def __iter__(self):
        native = getattr(self.dataset, "native_file", lambda: None)()
        if native is not None:
            C = _ext.load(required=False)
            batcher = C.TokenBatcher(native, self.batch_size, self.dataset.sequence_length, self.ddp_rank,
                                     self.ddp_world_size, self.prefetch_depth, self.pin)
            n = (batcher.num_batches - self.ddp_rank + self.ddp_world_size - 1) // self.ddp_world_size
            for _ in range(max(n, 0)):
                yield batcher.next()
            return
        for b in range(self.ddp_rank, self._num_batches(), self.ddp_world_size):
            yield self.batch(b)


class DeviceFeeder:
    """Moves the batches of a loader to the device with asynchronous copies, and keeps the copies
    ordered against the loader's buffer reuse.

    The prefetching loader hands out views of pinned ring slots that stay valid only until two
    further batches have been fetched (the worker thread then refills the slot).  A training loop that
    fetches several micro-batches ahead of the GPU (gradient accumulation with no host sync in
    between) could therefore have a slot refilled while its host-to-device copy has not run yet.
    ``next()`` records an event after each pair of copies and, before fetching a batch whose arrival
    frees a slot, waits on the host for the copy that read that slot.  Loaders without a ring
    (fresh tensors per batch) pay one cheap event per batch.
    """

    kSlotsInFlight = 2      # a slot handed out by call n may be refilled once call n + 2 has begun

    def __init__(self, batches, device: torch.device):
        self._it = iter(batches)
        self.device = device
        self._pending: List = []          # events of the copies whose source slot may still be live

    def next(self) -> Tuple[torch.Tensor, torch.Tensor]:
        cuda = self.device.type == "cuda"
        if cuda and len(self._pending) >= self.kSlotsInFlight:
            self._pending.pop(0).synchronize()
        x, y = next(self._it)
        if not cuda:
            return x.to(self.device), y.to(self.device)
        dx, dy = x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pending.append(ev)
        return dx, dy

    def skip(self, n: int) -> None:
        """Drops ``n`` batches (resume: fast-forward past what a checkpoint had consumed)."""
        for _ in range(n):
            next(self._it)

    __next__ = next

    def __iter__(self):
        return self
