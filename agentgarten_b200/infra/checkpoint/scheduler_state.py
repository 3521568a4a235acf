"""Saving and restoring scheduler / GradScaler *progress* only.

A resumed run keeps its own recipe: the learning-rate lambda, base LRs and scaler growth
settings of the current configuration win; a checkpoint contributes only how far the
schedule had advanced (``last_epoch``, ``_step_count``, the scaler's scale and growth
tracker).  Learning rates are then recomputed from the current recipe at that progress.

Parity: reference ``wm/infra/checkpoint/scheduler_state.py:26-160``.
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any

import torch

from .common import warn_rank0
from .optimizer_state import option_equal

__all__ = ["LAMBDA_LR_ADAPTER", "restore_closed_form_scheduler_progress",
           "restore_grad_scaler_progress", "restore_lambda_lr_progress", "scheduler_adapter_name",
           "scheduler_state_for_save"]

LAMBDA_LR_ADAPTER = "lambda_lr_v1"
_GENERIC = "lr_scheduler_v1:"


def scheduler_adapter_name(scheduler) -> str:
    if isinstance(scheduler, torch.optim.lr_scheduler.LambdaLR):
        return LAMBDA_LR_ADAPTER
    kind = type(scheduler)
    return f"{_GENERIC}{kind.__module__}.{kind.__qualname__}"


def scheduler_state_for_save(scheduler) -> dict[str, Any]:
    # The whole state dict is written (a LambdaLR's callable objects appear as their attribute
    # dicts under ``lr_lambdas``), which keeps the directory layout identical to the reference's;
    # restoring reads the progress fields only, the callables stay those of the current recipe.
    return {"adapter": scheduler_adapter_name(scheduler), "state": dict(scheduler.state_dict())}


def _apply_lrs(scheduler, lrs: list[float]) -> None:
    for group, lr in zip(scheduler.optimizer.param_groups, lrs, strict=True):
        group["lr"] = lr
    scheduler._last_lr = lrs


def restore_lambda_lr_progress(scheduler, loaded_state: Mapping[str, Any], saved_fields: set[str]) -> bool:
    if "last_epoch" not in saved_fields:
        return False
    scheduler.last_epoch = int(loaded_state["last_epoch"])
    if "_step_count" in saved_fields:
        scheduler._step_count = int(loaded_state["_step_count"])
    _apply_lrs(scheduler, [base * fn(scheduler.last_epoch)
                           for base, fn in zip(scheduler.base_lrs, scheduler.lr_lambdas, strict=True)])
    return True


def restore_closed_form_scheduler_progress(name: str, scheduler, loaded_state: Mapping[str, Any],
                                           saved_fields: set[str]) -> bool:
    if "last_epoch" not in saved_fields:
        return False
    closed_form = getattr(scheduler, "_get_closed_form_lr", None)
    if not callable(closed_form):
        warn_rank0(f"Scheduler '{name}' ({type(scheduler).__name__}) cannot recompute learning "
                   "rates from restored progress; keeping it fresh.")
        return False
    current = scheduler.state_dict()
    progress = {"last_epoch", "_step_count", "_last_lr", "_get_lr_called_within_step"}
    if any(not option_equal(loaded_state[f], current[f]) for f in (set(loaded_state) & set(current)) - progress):
        warn_rank0(f"Scheduler '{name}' resumed progress while keeping current recipe options.")
    scheduler.last_epoch = int(loaded_state["last_epoch"])
    if "_step_count" in saved_fields:
        scheduler._step_count = int(loaded_state["_step_count"])
    _apply_lrs(scheduler, list(closed_form()))
    return True


def restore_grad_scaler_progress(grad_scaler, current_state: Mapping[str, Any], loaded_state: Mapping[str, Any],
                                 saved_fields: set[str]) -> bool:
    have = [f for f in ("scale", "_growth_tracker") if f in saved_fields]
    if have and not current_state:
        warn_rank0("Checkpoint has enabled GradScaler progress while the current GradScaler is "
                   "disabled; keeping it disabled.")
        return False
    if not have or not current_state:
        return False
    merged = dict(current_state)
    for f in have:
        merged[f] = loaded_state[f]
    grad_scaler.load_state_dict(merged)
    recipe = ("growth_factor", "backoff_factor", "growth_interval")
    if any(f in saved_fields and not option_equal(loaded_state[f], current_state[f]) for f in recipe):
        warn_rank0("GradScaler resumed scale progress while keeping current growth/backoff settings.")
    return True
