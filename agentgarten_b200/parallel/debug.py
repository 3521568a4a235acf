"""Debug aids of the peer-memory paths.

``AGB200_POISON=1`` fills every buffer that peers write into (tensor-parallel input rows and
partial-sum slots, the receive halves of the all-to-all) with 0xFF bytes when it is allocated:
bf16 / fp16 / fp32 NaN.  A kernel that consumes a row before its producer has stored it then
yields non-finite values, which the non-finite consensus of the trainer and the finiteness
assertions of the tests catch, instead of zeros that look like data.  Counters are never
poisoned.  Together with the bounded waits (status word) and the work-list checks inside the
kernels (``kBadIndex``) this stands in for a race detector, which this package cannot run.
"""

from __future__ import annotations

import os

import torch

__all__ = ["enabled", "poison"]


def enabled() -> bool:
    return os.environ.get("AGB200_POISON", "0") == "1"


def poison(buffer: torch.Tensor) -> torch.Tensor:
    """Fill ``buffer`` with 0xFF bytes when poisoning is on; returns it either way."""
    if enabled() and buffer.numel():
        buffer.view(torch.uint8).fill_(0xFF)
    return buffer
