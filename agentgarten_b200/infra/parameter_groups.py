"""Selecting and grouping a module's parameters by regular expressions over their names.

A parameter can have several names (tied weights).  Everywhere in this file a pattern
"matches a parameter" when it *fully* matches at least one of the parameter's names.
"""

from __future__ import annotations

import re
from collections.abc import Iterable, Mapping, Sequence
from typing import Any

import torch

__all__ = ["PatternSet", "enable_only", "group_by_declarations", "split_matrices_from_vectors"]


class PatternSet:
    """A few regular expressions, given as one string or a sequence of strings."""

    def __init__(self, patterns: str | Iterable[str]) -> None:
        texts = (patterns,) if isinstance(patterns, str) else tuple(patterns)
        self.compiled = tuple(re.compile(text) for text in texts)

    def matches(self, names: Iterable[str]) -> bool:
        return any(expression.fullmatch(name) for name in names for expression in self.compiled)


def _names_of_trainable(module: torch.nn.Module) -> dict[torch.nn.Parameter, list[str]]:
    """Every trainable parameter (in ``named_parameters`` order) with all of its names."""
    names: dict[torch.nn.Parameter, list[str]] = {
        parameter: [] for _, parameter in module.named_parameters() if parameter.requires_grad}
    for name, parameter in module.named_parameters(remove_duplicate=False):
        if parameter in names:
            names[parameter].append(name)
    return names


def group_by_declarations(module: torch.nn.Module,
                          declarations: Sequence[Mapping[str, Any]] | None = None) -> list[dict[str, Any]]:
    """Optimizer parameter groups of the trainable parameters of ``module``.

    Each declaration is ``{"patterns": ..., **group options}``.  A parameter goes to the first
    declaration that matches it; declarations that match nothing produce no group; what no
    declaration claims forms a plain group that comes first.
    """
    names = _names_of_trainable(module)
    if not declarations:
        return [{"params": list(names)}]
    unclaimed = dict.fromkeys(names)
    claimed_groups = []
    for declaration in declarations:
        wanted = PatternSet(declaration["patterns"])
        members = [parameter for parameter in unclaimed if wanted.matches(names[parameter])]
        if not members:
            continue
        for parameter in members:
            del unclaimed[parameter]
        options = {key: value for key, value in declaration.items() if key != "patterns"}
        claimed_groups.append({**options, "params": members})
    leading = [{"params": list(unclaimed)}] if unclaimed else []
    return leading + claimed_groups


def split_matrices_from_vectors(groups: Sequence[Mapping[str, Any]]) -> list[dict[str, Any]]:
    """Every group becomes up to two with the same options: parameters of two or more
    dimensions (weight decay applies) and the rest (norm weights, biases)."""
    result = []
    for group in groups:
        options = {key: value for key, value in group.items() if key != "params"}
        for wanted in (True, False):
            members = [p for p in group["params"] if (p.ndim >= 2) is wanted]
            if members:
                result.append({**options, "params": members})
    return result


def enable_only(module: torch.nn.Module, patterns: str | Sequence[str]) -> None:
    """Freeze ``module`` except the parameters that ``patterns`` match."""
    wanted = PatternSet(patterns)
    module.requires_grad_(False)
    for name, parameter in module.named_parameters(remove_duplicate=False):
        if wanted.matches((name,)):
            parameter.requires_grad_(True)
