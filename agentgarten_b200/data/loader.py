"""Resumable, rank-sharded data loader.

Each epoch draws one permutation from ``seed + epoch``, trims (or pads) it to a multiple of
the world size, and gives rank ``r`` the indices ``r, r + world, ...``.  The loader keeps a
cursor ``(epoch, batch_offset)`` that is published *before* a batch is yielded, so a
checkpoint taken while the batch is being trained on resumes with the next one.  Creating a
new iterator invalidates older ones.  ``resume_signature`` describes the stream; a saved
cursor is only reused when the signature matches.

Parity: reference ``wm/data/loader.py:22-139``.
"""

from __future__ import annotations

from collections.abc import Callable, Iterator, Mapping
from typing import Any

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, Dataset

__all__ = ["StatefulDataLoader"]


class StatefulDataLoader:
    def __init__(self, dataset: Dataset[Any], *, batch_size: int,
                 collate_fn: Callable[[list[Any]], Any] | None = None, shuffle: bool = True,
                 seed: int = 0, num_workers: int = 0, prefetch_factor: int | None = 2,
                 pin_memory: bool = True, drop_last: bool = True) -> None:
        self.dataset = dataset
        self.batch_size = int(batch_size)
        self.collate_fn = collate_fn
        self.shuffle, self.seed = bool(shuffle), int(seed)
        self.num_workers = int(num_workers)
        self.prefetch_factor = prefetch_factor if self.num_workers else None
        self.pin_memory, self.drop_last = bool(pin_memory), bool(drop_last)
        on = dist.is_available() and dist.is_initialized()
        self.num_replicas = dist.get_world_size() if on else 1
        self.rank = dist.get_rank() if on else 0
        self.epoch = 0
        self.batch_offset = 0
        self._generation = 0

    # ------------------------------------------------------------------- sampling
    def _indices(self, epoch: int) -> list[int]:
        n = len(self.dataset)
        if self.shuffle:
            order = torch.randperm(n, generator=torch.Generator().manual_seed(self.seed + epoch)).tolist()
        else:
            order = list(range(n))
        world = self.num_replicas
        if self.drop_last:
            order = order[: n - n % world]
        elif n % world:
            order += order[: world - n % world]
        return order[self.rank::world]

    def _batches(self, epoch: int) -> list[list[int]]:
        mine = self._indices(epoch)
        size = self.batch_size
        batches = [mine[i:i + size] for i in range(0, len(mine), size)]
        if self.drop_last and batches and len(batches[-1]) < size:
            batches.pop()
        return batches

    def __len__(self) -> int:
        return len(self._batches(self.epoch))

    # ------------------------------------------------------------------ iteration
    def __iter__(self) -> Iterator[Any]:
        epoch, start = self.epoch, self.batch_offset
        self._generation += 1
        batches = self._batches(epoch)
        loader = DataLoader(self.dataset, batch_sampler=batches[start:], collate_fn=self.collate_fn,
                            num_workers=self.num_workers, prefetch_factor=self.prefetch_factor,
                            pin_memory=self.pin_memory and torch.cuda.is_available(),
                            generator=torch.Generator().manual_seed(self.seed + epoch))
        # workers start here, before callbacks create background threads
        return self._walk(iter(loader), epoch, start, len(batches), self._generation)

    def _walk(self, source: Iterator[Any], epoch: int, start: int, total: int, generation: int):
        for index, batch in enumerate(source, start=start):
            if generation != self._generation:
                raise RuntimeError("loader iterator superseded; call iter(loader) again")
            if index + 1 == total:
                self.epoch, self.batch_offset = epoch + 1, 0
            else:
                self.batch_offset = index + 1
            yield batch
        if self.epoch == epoch:
            self.epoch, self.batch_offset = epoch + 1, 0

    # ---------------------------------------------------------------------- state
    def resume_signature(self) -> dict[str, Any]:
        describe = getattr(self.dataset, "resume_signature", None)
        return {"dataset_size": len(self.dataset),
                "dataset": describe() if callable(describe) else None,
                "batch_size": self.batch_size, "shuffle": self.shuffle, "seed": self.seed,
                "drop_last": self.drop_last}

    def state_dict(self) -> dict[str, int]:
        return {"epoch": self.epoch, "batch_offset": self.batch_offset}

    def load_state_dict(self, state: Mapping[str, Any]) -> None:
        epoch, offset = int(state["epoch"]), int(state["batch_offset"])
        if epoch < 0 or offset < 0:
            raise ValueError(f"invalid loader cursor {dict(state)}")
        total = len(self._batches(epoch))
        if total and offset >= total:
            epoch, offset = epoch + offset // total, offset % total
        self.epoch, self.batch_offset = epoch, offset
        self._generation += 1
