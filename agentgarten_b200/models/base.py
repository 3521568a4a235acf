"""Objectives that train a generator against a frozen conditioner.

``ConditionedModel`` owns what every such objective shares: the conditioner (codec and text
tower) is frozen at construction and left out of checkpoints, raw batches are encoded by it
once they are on the training device, and sampling options are a closed set — a call may
override the configured values but not invent new keys.

Parity: reference ``wm/models/base.py:20-63`` (same public methods and checkpoint contract).
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any, ClassVar

from torch import nn

from agentgarten_b200.infra.model import Model
from agentgarten_b200.parallel.engine import ParallelConfig, parallelize_network

__all__ = ["ConditionedModel"]


class ConditionedModel(Model):
    # State-dict keys below these prefixes belong to frozen roles and are never saved;
    # subclasses with more frozen networks (a teacher, say) append theirs.
    checkpoint_excluded_prefixes: ClassVar[tuple[str, ...]] = ("conditioner.",)

    def __init__(self, *, conditioner: nn.Module, sampling_defaults: Mapping[str, Any],
                 sampling: Mapping[str, Any] | None = None) -> None:
        super().__init__()
        for parameter in conditioner.parameters():
            parameter.requires_grad_(False)
        self.conditioner = conditioner
        self.sampling: dict[str, Any] = dict(sampling_defaults)
        self.sampling.update(sampling or {})

    # -- placement ------------------------------------------------------------------------
    def parallelize_conditioner(self, config: ParallelConfig, device) -> None:
        """Only the text tower has weights worth placing; the codec loads itself lazily."""
        parallelize_network(self.conditioner.text_encoder, config, device)

    # -- data -----------------------------------------------------------------------------
    def prepare_data_batch(self, data_batch: dict[str, Any]) -> dict[str, Any]:
        return self.conditioner.encode(data_batch, training=self.training)

    # -- checkpoints ----------------------------------------------------------------------
    def checkpoint_model_state_dict(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        frozen = self.checkpoint_excluded_prefixes
        kept = {}
        for key, value in state_dict.items():
            if not key.startswith(frozen):
                kept[key] = value
        return kept

    # -- sampling -------------------------------------------------------------------------
    def sampling_options(self, overrides: Mapping[str, Any]) -> dict[str, Any]:
        """Configured options with per-call ``overrides``; unknown keys are an error."""
        stray = sorted(key for key in overrides if key not in self.sampling)
        if stray:
            raise TypeError(f"unknown sampling options {stray}")
        merged = dict(self.sampling)
        merged.update(overrides)
        return merged
