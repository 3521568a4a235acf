"""Learning-rate multipliers for ``torch.optim.lr_scheduler.LambdaLR``.

Plain picklable classes with keyword-only constructors, so a scheduler survives
checkpointing and a resolved ``config.yaml`` written by either implementation instantiates
here.  Keyword names, defaults and validation follow the reference
(``wm/infra/optim/lr.py:8-77``): ``LinearWarmup(warmup_steps=100, start_factor=1e-6)``,
``CosineDecay(decay_steps, min_factor=0)``, ``LinearWarmupCosineDecay(warmup_steps,
decay_steps, start_factor=0, min_factor=0)`` where ``decay_steps`` counts from step 0 and
includes the warm-up.
"""

from __future__ import annotations

import math

__all__ = ["CosineDecay", "LinearWarmup", "LinearWarmupCosineDecay"]


def _unit_interval(name: str, value: float) -> float:
    value = float(value)
    if not math.isfinite(value) or not 0.0 <= value <= 1.0:
        raise ValueError(f"{name} must be finite and in [0, 1]")
    return value


def _half_cosine(progress: float, floor: float) -> float:
    return floor + (1.0 - floor) * 0.5 * (1.0 + math.cos(math.pi * progress))


class LinearWarmup:
    """``start_factor`` → 1 over ``warmup_steps`` updates, then constant 1."""

    def __init__(self, *, warmup_steps: int = 100, start_factor: float = 1.0e-6) -> None:
        self.warmup_steps = int(warmup_steps)
        self.start_factor = float(start_factor)

    def __call__(self, step: int) -> float:
        if self.warmup_steps <= 0 or step >= self.warmup_steps:
            return 1.0
        ramp = max(float(step), 0.0) / float(self.warmup_steps)
        return self.start_factor + (1.0 - self.start_factor) * ramp


class CosineDecay:
    """1 → ``min_factor`` along half a cosine over ``decay_steps`` updates."""

    def __init__(self, *, decay_steps: int, min_factor: float = 0.0) -> None:
        self.decay_steps = int(decay_steps)
        if self.decay_steps <= 0:
            raise ValueError("decay_steps must be positive")
        self.min_factor = _unit_interval("min_factor", min_factor)

    def __call__(self, step: int) -> float:
        done = min(max(float(step), 0.0), float(self.decay_steps)) / float(self.decay_steps)
        return _half_cosine(done, self.min_factor)


class LinearWarmupCosineDecay:
    """Linear ramp to 1 at ``warmup_steps``, then half a cosine down to ``min_factor`` at
    ``decay_steps`` (both counted from step 0), constant afterwards."""

    def __init__(self, *, warmup_steps: int, decay_steps: int, start_factor: float = 0.0,
                 min_factor: float = 0.0) -> None:
        self.warmup_steps, self.decay_steps = int(warmup_steps), int(decay_steps)
        if self.warmup_steps < 0:
            raise ValueError("warmup_steps must be non-negative")
        if self.decay_steps <= self.warmup_steps:
            raise ValueError("decay_steps must be greater than warmup_steps")
        self.start_factor = _unit_interval("start_factor", start_factor)
        self.min_factor = _unit_interval("min_factor", min_factor)

    def __call__(self, step: int) -> float:
        at = min(max(float(step), 0.0), float(self.decay_steps))
        if self.warmup_steps and at < self.warmup_steps:
            return self.start_factor + (1.0 - self.start_factor) * at / float(self.warmup_steps)
        done = (at - self.warmup_steps) / float(self.decay_steps - self.warmup_steps)
        return _half_cosine(done, self.min_factor)
