"""Tensor-tree helpers, seeding and scoped module state.

Parity: reference ``wm/infra/utils.py:30-138``.
"""

from __future__ import annotations

import contextlib
import os
import random
from collections import defaultdict
from collections.abc import Callable, Iterator, Mapping, Sequence
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

__all__ = [
    "frozen_parameters",
    "map_tensors",
    "prefetch",
    "preserve_training_mode",
    "set_random_seed",
    "to",
]


def map_tensors(value: Any, transform: Callable[[torch.Tensor], torch.Tensor]) -> Any:
    """Rebuild a nested container with ``transform`` applied to every tensor.

    A tensor object that occurs several times is transformed once and stays one object in the
    result (a batch that shares a tensor between two keys still shares it after a device move).
    Mappings and sequences come back as their own types (default dictionaries keep their
    factory, named tuples their fields); strings, byte strings and ranges are leaves.
    Reference: ``wm/infra/utils.py:30-52``.
    """
    done: dict[int, torch.Tensor] = {}

    def visit(item: Any) -> Any:
        if isinstance(item, torch.Tensor):
            if id(item) not in done:
                done[id(item)] = transform(item)
            return done[id(item)]
        if isinstance(item, Mapping):
            children = {key: visit(child) for key, child in item.items()}
            if isinstance(item, defaultdict):
                return type(item)(item.default_factory, children)
            return type(item)(children)
        if isinstance(item, tuple) and hasattr(item, "_fields"):
            return type(item)(*(visit(child) for child in item))
        if isinstance(item, Sequence) and not isinstance(item, (str, bytes, bytearray, range)):
            return type(item)([visit(child) for child in item])
        return item

    return visit(value)


def to(data: Any, device: torch.device | str | None = None, dtype: torch.dtype | None = None,
       memory_format: torch.memory_format = torch.preserve_format) -> Any:
    """Move / cast every tensor of a tree.  Copies to an accelerator are asynchronous (the source
    may be pinned), copies to the host are not; a channels-last format is applied only to
    tensors of the matching rank (4 for ``channels_last``, 5 for ``channels_last_3d``)."""
    to_host = device is not None and torch.device(device).type == "cpu"
    rank_of = {torch.channels_last: 4, torch.channels_last_3d: 5}

    def move(tensor: torch.Tensor) -> torch.Tensor:
        layout = memory_format if rank_of.get(memory_format, tensor.dim()) == tensor.dim() \
            else torch.preserve_format
        return tensor.to(device=device, dtype=dtype, memory_format=layout, non_blocking=not to_host)

    return map_tensors(data, move)


def set_random_seed(seed: int, by_rank: bool = False) -> None:
    if by_rank and dist.is_available() and dist.is_initialized():
        seed = seed + dist.get_rank()
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)


@contextlib.contextmanager
def preserve_training_mode(model: torch.nn.Module) -> Iterator[None]:
    modes = {module: module.training for module in model.modules()}
    try:
        yield
    finally:
        for module, mode in modes.items():
            module.training = mode


@contextlib.contextmanager
def frozen_parameters(module: torch.nn.Module) -> Iterator[None]:
    """Temporarily mark all parameters as not requiring grad."""
    flags = [(p, p.requires_grad) for p in module.parameters()]
    try:
        for p, _ in flags:
            p.requires_grad_(False)
        yield
    finally:
        for p, flag in flags:
            p.requires_grad_(flag)


def prefetch(path: str | Path, *, threads: int = 16, chunk: int = 64 << 20) -> None:
    """Warm the page cache of ``path`` with parallel positional reads."""
    size = os.path.getsize(path)
    fd = os.open(path, os.O_RDONLY)
    try:
        def read(start: int) -> None:
            remaining = min(chunk, size - start)
            offset = start
            while remaining > 0:
                got = os.preadv(fd, [bytearray(min(remaining, 8 << 20))], offset)
                if got <= 0:
                    break
                offset += got
                remaining -= got

        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(read, range(0, size, chunk)))
    finally:
        os.close(fd)
