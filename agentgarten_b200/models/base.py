"""Shared lifecycle of objectives that train against a frozen conditioner.

Parity: reference ``wm/models/base.py:20-63``.
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any, ClassVar

import torch
from torch import nn

from agentgarten_b200.infra.model import Model
from agentgarten_b200.parallel.engine import ParallelConfig, parallelize_network

__all__ = ["ConditionedModel"]


class ConditionedModel(Model):
    """The conditioner (codec + text tower) is never trained and never checkpointed.

    Subclasses with further frozen roles extend ``checkpoint_excluded_prefixes``.
    """

    checkpoint_excluded_prefixes: ClassVar[tuple[str, ...]] = ("conditioner.",)

    def __init__(self, *, conditioner: nn.Module, sampling_defaults: Mapping[str, Any],
                 sampling: Mapping[str, Any] | None = None) -> None:
        super().__init__()
        self.conditioner = conditioner
        self.conditioner.requires_grad_(False)
        self.sampling: dict[str, Any] = {**sampling_defaults, **dict(sampling or {})}

    def parallelize_conditioner(self, config: ParallelConfig, device) -> None:
        parallelize_network(self.conditioner.text_encoder, config, device)

    def prepare_data_batch(self, data_batch: dict[str, Any]) -> dict[str, Any]:
        return self.conditioner.encode(data_batch, training=self.training)

    def checkpoint_model_state_dict(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        skip = self.checkpoint_excluded_prefixes
        return {k: v for k, v in state_dict.items() if not k.startswith(skip)}

    def sampling_options(self, overrides: Mapping[str, Any]) -> dict[str, Any]:
        unknown = set(overrides) - set(self.sampling)
        if unknown:
            raise TypeError(f"unknown sampling options {sorted(unknown)}")
        return {**self.sampling, **overrides}
