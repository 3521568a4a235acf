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


class _ClosedOptions(dict):
    """Options whose key set is fixed when the model is built: a call may change values, not
    add keys (a misspelt option must not be ignored silently for a whole sampling run)."""

    def overridden(self, changes: Mapping[str, Any]) -> dict[str, Any]:
        merged = dict(self)
        for key, value in changes.items():
            if key not in merged:
                stray = sorted(name for name in changes if name not in self)
                raise TypeError(f"unknown sampling options {stray}")
            merged[key] = value
        return merged


class ConditionedModel(Model):
    # State-dict keys below these prefixes belong to frozen roles and are never saved;
    # subclasses with more frozen networks (a teacher, say) list theirs as well.
    checkpoint_excluded_prefixes: ClassVar[tuple[str, ...]] = ("conditioner.",)

    def __init__(self, *, conditioner: nn.Module, sampling_defaults: Mapping[str, Any],
                 sampling: Mapping[str, Any] | None = None) -> None:
        super().__init__()
        self.conditioner = conditioner.requires_grad_(False)
        self.sampling = _ClosedOptions(sampling_defaults)
        self.sampling.update(sampling or {})

    def parallelize_conditioner(self, config: ParallelConfig, device) -> None:
        """Only the text tower has weights worth placing; the codec loads itself lazily."""
        parallelize_network(self.conditioner.text_encoder, config, device)

    def prepare_data_batch(self, data_batch: dict[str, Any]) -> dict[str, Any]:
        """Raw batch -> latents and token ids, on the training device (cached keys pass through)."""
        return self.conditioner.encode(data_batch, training=self.training)

    def checkpoint_model_state_dict(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        frozen = self.checkpoint_excluded_prefixes
        return dict(item for item in state_dict.items() if not item[0].startswith(frozen))

    def sampling_options(self, overrides: Mapping[str, Any]) -> dict[str, Any]:
        """Configured options with per-call ``overrides``; unknown keys are a ``TypeError``."""
        return self.sampling.overridden(overrides)
