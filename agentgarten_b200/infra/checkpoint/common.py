"""Small helpers shared by the checkpoint modules."""

from __future__ import annotations

import warnings
from typing import Any

import torch.distributed as dist

TENSOR_COMPONENTS = ("model", "optimizers", "schedulers", "trainer")
ALL_COMPONENTS = (*TENSOR_COMPONENTS, "dataloader")


def rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def warn_rank0(message: str) -> None:
    if rank() == 0:
        warnings.warn(message, stacklevel=3)


def gather_objects(value: Any) -> list[Any]:
    if world_size() == 1:
        return [value]
    out: list[Any] = [None] * world_size()
    dist.all_gather_object(out, value)
    return out


def brief(error: BaseException | None) -> str | None:
    if error is None:
        return None
    return f"{type(error).__name__}: {' '.join(str(error).split())[:400]}"


def raise_together(stage: str, local_error: BaseException | None) -> None:
    """If any rank failed in ``stage``, raise on every rank (with all messages)."""
    reports = gather_objects(brief(local_error))
    failed = [(r, m) for r, m in enumerate(reports) if m is not None]
    if failed:
        detail = "; ".join(f"rank {r}: {m}" for r, m in failed)
        raise RuntimeError(f"Checkpoint {stage} failed: {detail}") from local_error
