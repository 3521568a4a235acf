"""Named ranges for timelines: NVTX on CUDA when ``AGB200_NVTX=1``, nothing otherwise.

The reference has no tracing.  Here the trainer phases (data, forward/backward, optimizer),
the fused layer (forward, backward) and the tensor-parallel phases are wrapped in ranges, so
an Nsight Systems timeline of a step reads like the call structure.  With the variable
unset a span costs one attribute lookup.
"""

from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Iterator

import torch

__all__ = ["enabled", "span"]

_ON = os.environ.get("AGB200_NVTX") == "1"


def enabled() -> bool:
    return _ON and torch.cuda.is_available()


@contextmanager
def span(name: str) -> Iterator[None]:
    if not enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
