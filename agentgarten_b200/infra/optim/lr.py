"""Learning-rate multipliers for ``torch.optim.lr_scheduler.LambdaLR``.

Picklable callables (plain classes), so schedulers survive checkpointing and the resolved
configuration round-trips through YAML.

Parity: reference ``wm/infra/optim/lr.py:8-77``.
"""

from __future__ import annotations

import math

__all__ = ["CosineDecay", "LinearWarmup", "LinearWarmupCosineDecay"]


class LinearWarmup:
    """``start_factor`` → 1 over ``warmup_steps`` updates, then constant 1."""

    def __init__(self, warmup_steps: int, start_factor: float = 0.0) -> None:
        if warmup_steps < 0:
            raise ValueError("warmup_steps must be non-negative")
        self.warmup_steps, self.start_factor = int(warmup_steps), float(start_factor)

    def __call__(self, step: int) -> float:
        if self.warmup_steps == 0 or step >= self.warmup_steps:
            return 1.0
        return self.start_factor + (1.0 - self.start_factor) * step / self.warmup_steps


class CosineDecay:
    """1 → ``final_factor`` along half a cosine over ``total_steps``."""

    def __init__(self, total_steps: int, final_factor: float = 0.0) -> None:
        if total_steps <= 0:
            raise ValueError("total_steps must be positive")
        self.total_steps, self.final_factor = int(total_steps), float(final_factor)

    def __call__(self, step: int) -> float:
        progress = min(max(step, 0), self.total_steps) / self.total_steps
        return self.final_factor + (1.0 - self.final_factor) * 0.5 * (1.0 + math.cos(math.pi * progress))


class LinearWarmupCosineDecay:
    def __init__(self, warmup_steps: int, total_steps: int, start_factor: float = 0.0,
                 final_factor: float = 0.0) -> None:
        if total_steps <= warmup_steps:
            raise ValueError("total_steps must exceed warmup_steps")
        self.warmup = LinearWarmup(warmup_steps, start_factor)
        self.decay = CosineDecay(total_steps - warmup_steps, final_factor)
        self.warmup_steps = int(warmup_steps)

    def __call__(self, step: int) -> float:
        if step < self.warmup_steps:
            return self.warmup(step)
        return self.decay(step - self.warmup_steps)
