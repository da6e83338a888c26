"""Resumable, rank-aware data loading (reference: ``areal/utils/dataloader.py`` —
``StatefulDataLoader`` + ``DistributedSampler``).

:class:`StatefulDataLoader` walks a map-style dataset in a permutation that depends only on
``(seed, epoch)``; every data-parallel rank takes a strided slice of it, so the ranks see
disjoint samples and the same number of batches. ``state_dict`` records the epoch and how many
batches of it were handed out; after ``load_state_dict`` iteration resumes with the next batch
of the same permutation (what the recover checkpoint needs to not repeat or skip data).
"""
from __future__ import annotations

from typing import Any, Callable, Iterator, Optional

import torch


class StatefulDataLoader:
    def __init__(self, dataset, batch_size: int, shuffle: bool = True, drop_last: bool = True, collate_fn: Optional[Callable] = None,
                 seed: int = 0, rank: int = 0, world_size: int = 1):
        if batch_size <= 0:
            raise ValueError("batch_size must be positive")
        self.dataset, self.batch_size, self.shuffle, self.drop_last = dataset, batch_size, shuffle, drop_last
        self.collate_fn = collate_fn or (lambda items: items)
        self.seed, self.rank, self.world_size = seed, rank, world_size
        self.epoch = 0
        self._served = 0          # batches of the current epoch already handed out
        self._resume_from = 0

    # ---- sizes
    def _per_rank(self) -> int:
        n = len(self.dataset)
        return n // self.world_size if self.drop_last else -(-n // self.world_size)

    def __len__(self) -> int:
        n = self._per_rank()
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)

    # ---- order
    def _indices(self, epoch: int) -> list[int]:
        n = len(self.dataset)
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed * 1000003 + epoch)
            order = torch.randperm(n, generator=g).tolist()
        else:
            order = list(range(n))
        per = self._per_rank()
        if not self.drop_last and per * self.world_size > n:      # pad by wrapping so every rank has `per` samples
            order += order[: per * self.world_size - n]
        return order[self.rank: per * self.world_size: self.world_size]

    def __iter__(self) -> Iterator[Any]:
        idx = self._indices(self.epoch)
        nb = len(self)
        start, self._resume_from = self._resume_from, 0
        self._served = start
        for b in range(start, nb):
            chunk = idx[b * self.batch_size:(b + 1) * self.batch_size]
            self._served = b + 1
            yield self.collate_fn([self.dataset[i] for i in chunk])
        self.epoch += 1
        self._served = 0

    # ---- checkpointing
    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "served": self._served, "seed": self.seed, "world_size": self.world_size}

    def load_state_dict(self, sd: dict) -> None:
        if sd.get("world_size", self.world_size) != self.world_size:
            raise ValueError("dataloader state was saved with a different data-parallel size")
        self.epoch = int(sd["epoch"])
        self._resume_from = int(sd.get("served", 0))
        if self._resume_from >= len(self):       # the epoch was complete
            self.epoch += 1
            self._resume_from = 0
        self.seed = int(sd.get("seed", self.seed))


def create_dataloader(dataset, batch_size: int, rank: int = 0, world_size: int = 1, shuffle: bool = True, drop_last: bool = True,
                      collate_fn: Optional[Callable] = None, seed: int = 0) -> StatefulDataLoader:
    """``batch_size`` is the GLOBAL batch; every rank draws ``batch_size // world_size`` samples per step."""
    if batch_size % world_size:
        raise ValueError(f"global batch size {batch_size} is not divisible by the {world_size} data-parallel ranks")
    return StatefulDataLoader(dataset, batch_size // world_size, shuffle, drop_last, collate_fn, seed, rank, world_size)
