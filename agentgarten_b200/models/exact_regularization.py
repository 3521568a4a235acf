"""Exact R1/R2 gradient penalties of a head ``h`` on a frozen feature backbone ``f``.

With ``D(x) = h(f(x))`` the penalty of a row is ``R = ||∇ₓD||²``.  Its gradient with
respect to the head parameters is obtained without differentiating the backbone twice:

1. ``u = ∇ₓD`` by reverse mode through the frozen backbone and the (frozen) head.
2. ``t = J_f(x)·u`` by forward mode through the backbone only (no graph is kept; attention
   contributes through its JVP operator).
3. ``⟨∇_φ h(φ), t⟩`` at ``φ = f(x)`` equals ``uᵀu = R`` and is differentiable with respect to
   the head: a double backward through the small head only.  ``dR/dθ = 2·d⟨∇_φ h, t⟩/dθ``.

The returned surrogate has value zero and carries exactly that gradient.

Parity: reference ``wm/models/exact_regularization.py:28-74``.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch
import torch.autograd.forward_ad as fwAD
from torch import Tensor, nn

from agentgarten_b200.utils.misc import frozen_parameters

__all__ = ["ExactPenalty", "check_exact_regularization", "exact_penalties"]

FeatureFunction = Callable[[Tensor], tuple[Tensor, ...]]


@dataclass
class ExactPenalty:
    logits: Tensor     # [N], differentiable w.r.t. the head
    penalty: Tensor    # [N], ||∇ₓD||² per row (detached)
    surrogate: Tensor  # [N], value 0, gradient dR/dθ


def exact_penalties(features: FeatureFunction, head: nn.Module, rows: Tensor) -> ExactPenalty:
    wide = torch.promote_types(rows.dtype, torch.float32)
    # (1) input gradient
    leaf = rows.detach().requires_grad_(True)
    with frozen_parameters(head), torch.enable_grad():
        (direction,) = torch.autograd.grad(head([features(leaf)]).sum(), leaf)
    direction = direction.detach()
    # (2) feature tangents along it
    with torch.no_grad(), fwAD.dual_level():
        duals = features(fwAD.make_dual(rows.detach(), direction.to(rows.dtype)))
        pairs = [fwAD.unpack_dual(d) for d in duals]
        primals = tuple(p.primal.detach() for p in pairs)
        tangents = tuple(torch.zeros_like(p.primal) if p.tangent is None else p.tangent.detach()
                         for p in pairs)
    # (3) directional derivative of the head, differentiable w.r.t. its parameters
    with torch.enable_grad():
        inputs = [p.requires_grad_(True) for p in primals]
        logits = head([inputs])
        grads = torch.autograd.grad(logits.sum(), inputs, create_graph=True)
        directional = sum((g.to(wide) * t.to(wide)).flatten(1).sum(1)
                          for g, t in zip(grads, tangents, strict=True))
    surrogate = 2.0 * directional
    return ExactPenalty(logits=logits,
                        penalty=direction.to(wide).square().flatten(1).sum(1),
                        surrogate=surrogate - surrogate.detach())


def check_exact_regularization(real_score: nn.Module, discriminator: nn.Module) -> None:
    if any(p.requires_grad for p in real_score.parameters()):
        raise ValueError("exact R1/R2 requires a frozen real score")
    if not isinstance(getattr(discriminator, "feature_layers", None), Sequence):
        raise TypeError("exact R1/R2 needs a discriminator exposing feature_layers")
