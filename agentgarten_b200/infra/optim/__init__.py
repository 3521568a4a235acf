"""Optimizers and learning-rate schedules."""

from .fused_adam import FusedAdam
from .lr import CosineDecay, LinearWarmup, LinearWarmupCosineDecay

__all__ = ["CosineDecay", "FusedAdam", "LinearWarmup", "LinearWarmupCosineDecay"]
