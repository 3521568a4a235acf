"""Experiment selection and command-line overrides.

``compose_config(["experiment=cosmos3/bidirectional", "trainer.grad_accum_steps=2", ...])``
imports ``<experiment_module_root>.cosmos3.bidirectional``, calls its ``build_config()``,
applies the remaining overrides, resolves interpolations and fails on missing (``???``)
values.  Exactly one plain ``experiment=family/name`` selector is required.

Parity: reference ``wm/configs/compose.py:21-81`` (built on hydra there).
"""

from __future__ import annotations

import importlib
from collections.abc import Sequence

from agentgarten_b200.infra.config import ConfigNode, LazyDict, apply_overrides, parse_override, resolve

__all__ = ["EXPERIMENT_MODULE_ROOT", "compose_config"]

EXPERIMENT_MODULE_ROOT = "agentgarten_b200.configs.experiments"


def _selector(overrides: Sequence[str]) -> tuple[str, list]:
    parsed = [parse_override(text) for text in overrides]
    chosen = [o for o in parsed if o.key == "experiment"]
    if len(chosen) != 1:
        raise ValueError("Exactly one plain experiment=... selector is required")
    only = chosen[0]
    if only.kind != "set" or not isinstance(only.value, str):
        raise ValueError("experiment must be a single plain scalar selector")
    return only.value, [o for o in parsed if o.key != "experiment"]


def _module_name(selector: str, root: str) -> str:
    parts = selector.split("/")
    if len(parts) < 2 or any(not p.isidentifier() for p in parts):
        raise ValueError("experiment must be an importable path such as family/name or "
                         "family/objective/version")
    return ".".join((root, *parts))


def compose_config(overrides: Sequence[str], *, experiment_module_root: str = EXPERIMENT_MODULE_ROOT,
                   ) -> LazyDict:
    selector, rest = _selector(overrides)
    if experiment_module_root == "wm.configs.experiments":
        experiment_module_root = EXPERIMENT_MODULE_ROOT
    module = importlib.import_module(_module_name(selector, experiment_module_root))
    builder = getattr(module, "build_config", None)
    if not callable(builder):
        raise TypeError(f"{module.__name__}.build_config is not callable")
    config = builder()
    if not isinstance(config, ConfigNode):
        raise TypeError(f"{module.__name__}.build_config() must return LazyDict")
    config["experiment"] = selector
    apply_overrides(config, rest)
    return resolve(config, throw_on_missing=True)
