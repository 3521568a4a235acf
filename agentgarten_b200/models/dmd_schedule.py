"""Configuration objects of the Adversarial Forcing objective: rollout endpoints, the GAN
term's weights and regulariser, and the clock that assigns a role to every iteration.

Parity: reference ``wm/models/dmd.py:55-140`` (field names, defaults, cadence rule).
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import StrEnum

__all__ = ["RCM_ENDPOINTS", "GANConfig", "PhaseClock", "Regularization"]

# Noise levels at which a block is queried during the few-step rollout (an n-step rollout uses
# the first n): 1 - 1/1601, 1 - 1/16, 1 - 1/6, 1 - 3/8.
RCM_ENDPOINTS = (1600.0 / 1601.0, 15.0 / 16.0, 5.0 / 6.0, 5.0 / 8.0)


class Regularization(StrEnum):
    FINITE_DIFFERENCE = "finite_difference"   # E[(D(x + sigma eps) - D(x))^2]
    EXACT = "exact"                           # E[|grad_x D|^2], exact gradient to the head


@dataclass(frozen=True)
class GANConfig:
    generator_weight: float = 0.01
    discriminator_weight: float = 0.01
    relativistic: bool = True
    regularization: Regularization = Regularization.FINITE_DIFFERENCE
    regularization_weight: float = 30.0        # finite difference
    regularization_sigma: float = 0.05
    exact_regularization_weight: float = 0.075  # = 30 * 0.05^2: the same local scale
    warmup_updates: int = 0                    # discriminator-only iterations at the start

    def __post_init__(self) -> None:
        object.__setattr__(self, "regularization", Regularization(self.regularization))
        if self.warmup_updates < 0:
            raise ValueError("warmup_updates must be non-negative")


@dataclass(frozen=True)
class PhaseClock:
    """After ``warmup_updates`` discriminator-only iterations, cycles of one student update
    followed by ``fake_score_updates_per_student`` fake-score (and discriminator) updates."""

    fake_score_updates_per_student: int = 5
    warmup_updates: int = 0

    def __post_init__(self) -> None:
        if self.fake_score_updates_per_student < 1 or self.warmup_updates < 0:
            raise ValueError(f"invalid phase clock {self}")

    @property
    def cycle(self) -> int:
        return 1 + self.fake_score_updates_per_student

    def _position(self, iteration: int) -> int | None:
        """Index inside the current cycle (0 = the student's turn), ``None`` during warm-up."""
        past = iteration - self.warmup_updates
        return None if past < 0 else past % self.cycle

    def is_warmup(self, iteration: int) -> bool:
        return self._position(iteration) is None

    def is_student(self, iteration: int) -> bool:
        return self._position(iteration) == 0

    def role_updates(self, iteration: int) -> dict[str, int]:
        """How many updates each role has had once ``iteration`` iterations are complete."""
        past = max(iteration - self.warmup_updates, 0)
        full, partial = divmod(past, self.cycle)
        student = full + (1 if partial else 0)
        return {"student": student, "fake_score": past - student}

    def is_cadence_due(self, iteration: int, interval: int | None) -> bool:
        """Periodic work (checkpoints, validation) is counted in student updates and fires only
        where a whole cycle has just finished, so both roles are at a consistent point."""
        if not interval or interval < 0 or iteration <= 0:
            return False
        done = self.role_updates(iteration)
        per_student = self.fake_score_updates_per_student
        return (done["student"] > 0 and done["fake_score"] > 0
                and done["student"] % interval == 0
                and done["fake_score"] % (interval * per_student) == 0)
