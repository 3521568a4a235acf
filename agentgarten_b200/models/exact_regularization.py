"""Exact R1/R2 gradient penalties of a head ``h`` on a frozen feature backbone ``f``.

The discriminator is ``D(x) = h(f(x))`` and the penalty of one row is ``R(x) = |∇ₓD|²``.  What
training needs is ``dR/dθ`` for the head's parameters ``θ``.  Differentiating the backbone
twice is avoided by three passes:

``u = ∇ₓD``
    reverse mode through backbone and head, everything frozen.
``t = J_f(x) · u``
    forward mode through the backbone alone, no graph kept (attention contributes through its
    JVP operator).
``s(θ) = ⟨∇_φ h_θ(φ), t⟩`` at ``φ = f(x)``
    equals ``uᵀu = R`` at the current ``θ`` and depends on ``θ`` through the small head only;
    ``dR/dθ = 2 ds/dθ`` needs a double backward through the head, nothing more.

``exact_penalties`` returns the logits, the penalty values and a *surrogate* whose value is zero
and whose gradient is exactly ``dR/dθ`` per row.

Parity: reference ``wm/models/exact_regularization.py:28-74``.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch
import torch.autograd.forward_ad as forward_mode
from torch import Tensor, nn

from agentgarten_b200.utils.misc import frozen_parameters

__all__ = ["ExactPenalty", "check_exact_regularization", "exact_penalties"]

FeatureFunction = Callable[[Tensor], tuple[Tensor, ...]]


@dataclass
class ExactPenalty:
    logits: Tensor     # [N], differentiable w.r.t. the head
    penalty: Tensor    # [N], |∇ₓD|² per row (detached)
    surrogate: Tensor  # [N], value 0, gradient dR/dθ


def _input_gradient(features: FeatureFunction, head: nn.Module, rows: Tensor) -> Tensor:
    probe = rows.detach().requires_grad_(True)
    with frozen_parameters(head), torch.enable_grad():
        (gradient,) = torch.autograd.grad(head([features(probe)]).sum(), probe)
    return gradient.detach()


def _pushed_forward(features: FeatureFunction, rows: Tensor, direction: Tensor):
    """``(f(x), J_f(x)·direction)`` for every feature tensor, both detached."""
    with torch.no_grad(), forward_mode.dual_level():
        outputs = features(forward_mode.make_dual(rows.detach(), direction.to(rows.dtype)))
        values, tangents = [], []
        for output in outputs:
            value, tangent = forward_mode.unpack_dual(output)
            values.append(value.detach())
            tangents.append(torch.zeros_like(value) if tangent is None else tangent.detach())
    return values, tangents


def exact_penalties(features: FeatureFunction, head: nn.Module, rows: Tensor) -> ExactPenalty:
    wide = torch.promote_types(rows.dtype, torch.float32)
    direction = _input_gradient(features, head, rows)
    values, tangents = _pushed_forward(features, rows, direction)
    with torch.enable_grad():
        leaves = [value.requires_grad_(True) for value in values]
        logits = head([leaves])
        slopes = torch.autograd.grad(logits.sum(), leaves, create_graph=True)
        along = sum((slope.to(wide) * tangent.to(wide)).flatten(1).sum(1)
                    for slope, tangent in zip(slopes, tangents, strict=True))
    doubled = 2.0 * along
    return ExactPenalty(logits=logits, penalty=direction.to(wide).square().flatten(1).sum(1),
                        surrogate=doubled - doubled.detach())


def check_exact_regularization(real_score: nn.Module, discriminator: nn.Module) -> None:
    """The scheme assumes a frozen backbone and a head that names the layers it taps."""
    if any(parameter.requires_grad for parameter in real_score.parameters()):
        raise ValueError("exact R1/R2 requires a frozen real score")
    if not isinstance(getattr(discriminator, "feature_layers", None), Sequence):
        raise TypeError("exact R1/R2 needs a discriminator exposing feature_layers")
