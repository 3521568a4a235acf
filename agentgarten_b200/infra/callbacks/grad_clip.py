"""Global-norm gradient clipping across optimizer roles.

The norm of a role is taken over the *reduced* gradient.  Optimizers that run the flat
sharded engine already have it: their reduce-scatter kernel emits the squared norm as a
side output, and clipping is applied by handing the coefficient (a device scalar) to the
fused Adam kernel instead of rescaling every gradient in memory.  Other optimizers are
measured with a foreach norm and clipped in place.  ``max_norm = inf`` only observes.

Parity: reference ``wm/infra/callbacks/grad_clip.py:24-112``.
"""

from __future__ import annotations

import math
from collections.abc import Iterable, Mapping
from typing import Any

import torch

from .base import Callback

__all__ = ["GradClip", "clip_grad_norm_", "clip_grad_norm_groups_", "clip_optimizers_"]


def _check(max_norm: float) -> float:
    value = float(max_norm)
    if math.isnan(value) or value < 0:
        raise ValueError("max_norm must be non-negative and not NaN")
    return value


def _live(parameters: Iterable[torch.Tensor], seen: set[int]) -> list[torch.Tensor]:
    out = []
    for p in parameters:
        if id(p) in seen:
            continue
        seen.add(id(p))
        if p.requires_grad and p.grad is not None:
            out.append(p)
    return out


@torch.no_grad()
def clip_grad_norm_groups_(parameter_groups: Mapping[str, Iterable[torch.Tensor]], max_norm: float):
    """Clip plain (non-engine) gradients in place; returns ``(total_norm, {role: norm})``."""
    max_norm = _check(max_norm)
    seen: set[int] = set()
    by_role = {str(role): _live(params, seen) for role, params in parameter_groups.items()}
    by_role = {role: params for role, params in by_role.items() if params}
    if not by_role:
        return None, {}
    role_norms = {}
    for role, params in by_role.items():
        norm = torch.nn.utils.get_total_norm([p.grad for p in params], norm_type=2.0,
                                             error_if_nonfinite=False)
        if hasattr(norm, "full_tensor"):
            norm = norm.full_tensor()
        role_norms[role] = norm.reshape(()).float()
    device = next(iter(role_norms.values())).device
    total = torch.linalg.vector_norm(torch.stack([n.to(device) for n in role_norms.values()]), ord=2.0)
    if not math.isinf(max_norm):
        everything = [p for params in by_role.values() for p in params]
        torch.nn.utils.clip_grads_with_norm_(everything, max_norm, total)
    return total, role_norms


@torch.no_grad()
def clip_grad_norm_(parameters: Iterable[torch.Tensor], max_norm: float):
    total, _ = clip_grad_norm_groups_({"model": parameters}, max_norm)
    return total


@torch.no_grad()
def clip_optimizers_(optimizers: Mapping[str, Any], max_norm: float):
    """Clip the gradients owned by named optimizers as one atomic update.

    Returns ``(total_norm, {role: norm}, coefficient)`` with device tensors; ``None`` norm
    when nothing has a gradient.  Engine-backed optimizers receive the coefficient through
    ``optimizer.grad_scale``; the rest are scaled in place.
    """
    max_norm = _check(max_norm)
    squares: dict[str, torch.Tensor] = {}
    plain: dict[str, list[torch.Tensor]] = {}
    seen: set[int] = set()
    for role, optimizer in optimizers.items():
        if getattr(optimizer, "engine", None) is not None:
            squares[str(role)] = optimizer.grad_norm_sq().float()
            continue
        reduce = getattr(optimizer, "reduce_gradients", None)
        if callable(reduce):
            reduce()
        params = _live((p for g in optimizer.param_groups for p in g["params"]), seen)
        if params:
            plain[str(role)] = params
            norms = torch._foreach_norm([p.grad for p in params], 2.0)
            squares[str(role)] = torch.stack([n.float() for n in norms]).square().sum()
    if not squares:
        return None, {}, None
    device = next(iter(squares.values())).device
    role_norms = {role: sq.to(device).sqrt() for role, sq in squares.items()}
    total = torch.stack([sq.to(device) for sq in squares.values()]).sum().sqrt()
    if math.isinf(max_norm):
        return total, role_norms, torch.ones((), device=device)
    coefficient = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for role, optimizer in optimizers.items():
        if getattr(optimizer, "engine", None) is not None:
            optimizer.grad_scale = coefficient
    for params in plain.values():
        torch._foreach_mul_([p.grad for p in params], coefficient.to(params[0].grad.device))
    return total, role_norms, coefficient


class GradClip(Callback):
    def __init__(self, max_norm: float = 1.0) -> None:
        super().__init__()
        self.max_norm = _check(max_norm)

    def on_before_optimizer_step(self, model_ddp, optimizer, scheduler, grad_scaler, iteration=0):
        del scheduler, grad_scaler, iteration
        clip_optimizers_({"net": optimizer}, self.max_norm)
