"""Which saved tensor goes into which live parameter.

Two modes.  *Strict-ish* (resume): a saved key restores the live key of the same name;
missing and unexpected keys are reported.  *Overlay* (initialisation from another model):
saved keys under ``source_prefix`` that fully match one of ``source_patterns`` are mapped to
``destination_prefix + key`` for one or many destination prefixes (e.g. the same released
tower into ``student``, ``real_score`` and ``fake_score``).  Two sources for one destination
are an error.  ``plan_model_initializations`` turns the ``train.model_initializations``
config section into an ordered list of overlay loads, merging consecutive entries that read
the same source.

Parity: reference ``wm/infra/checkpoint/plan.py:12-248``.
"""

from __future__ import annotations

import re
import warnings
from collections.abc import Iterable, Mapping, Sequence
from dataclasses import dataclass, replace
from typing import Any

from .common import raise_together

__all__ = ["ModelInitialization", "ModelLoadEntry", "ModelRestorePlan", "build_model_restore_plan",
           "model_prefix", "plan_model_initializations", "validate_overlay_target_shapes"]


def model_prefix(value: str | None) -> str:
    text = "" if value is None else str(value).strip(".")
    return f"{text}." if text else ""


@dataclass(frozen=True, slots=True)
class ModelLoadEntry:
    source_key: str
    targets: tuple[str, ...]

    @property
    def template_key(self) -> str:
        return self.targets[0]


@dataclass(frozen=True, slots=True)
class ModelRestorePlan:
    entries: tuple[ModelLoadEntry, ...]
    checkpoint_model_keys: frozenset[str]
    missing_model_keys: tuple[str, ...]
    unexpected_model_keys: tuple[str, ...]


def build_model_restore_plan(*, live_keys: Iterable[str], saved_keys: Iterable[str], overlay: bool,
                             source_prefix: str | None = None,
                             destination_prefixes: Sequence[str | None] = (None,),
                             source_patterns: Sequence[Any] = ()) -> ModelRestorePlan:
    live_order = tuple(live_keys)
    live, saved = set(live_order), set(saved_keys)
    if not overlay:
        return ModelRestorePlan(
            entries=tuple(ModelLoadEntry(k, (k,)) for k in live_order if k in saved),
            checkpoint_model_keys=frozenset(saved),
            missing_model_keys=tuple(sorted(live - saved)),
            unexpected_model_keys=tuple(sorted(saved - live)))
    source = model_prefix(source_prefix)
    destinations = tuple(dict.fromkeys(model_prefix(p) for p in destination_prefixes))
    if not destinations:
        raise ValueError("checkpoint overlay requires at least one destination")
    patterns = [re.compile(p) if isinstance(p, str) else p for p in source_patterns]
    chosen = sorted(k for k in saved if k.startswith(source) and (
        not patterns or any(p.fullmatch(k[len(source):]) for p in patterns)))
    in_scope = {k for k in live if k.startswith(destinations)}
    mapped: set[str] = set()
    origin: dict[str, str] = {}
    entries = []
    for key in chosen:
        targets = tuple(d + key[len(source):] for d in destinations)
        mapped.update(targets)
        present = tuple(t for t in targets if t in live)
        for t in present:
            before = origin.setdefault(t, key)
            if before != key:
                raise ValueError(f"Ambiguous checkpoint overlay for {t!r}: both {before!r} and "
                                 f"{key!r} map to it")
        if present:
            entries.append(ModelLoadEntry(key, present))
    return ModelRestorePlan(entries=tuple(entries), checkpoint_model_keys=frozenset(mapped),
                            missing_model_keys=tuple(sorted(in_scope - mapped)),
                            unexpected_model_keys=tuple(sorted(mapped - in_scope)))


def validate_overlay_target_shapes(plan: ModelRestorePlan, live_state: Mapping[str, Any]) -> None:
    """All destinations of one source tensor must agree in shape (checked on every rank)."""
    error: Exception | None = None
    for entry in plan.entries:
        shapes = {tuple(live_state[t].shape) for t in entry.targets}
        if len(shapes) > 1:
            error = ValueError(f"overlay source {entry.source_key!r} maps to destinations of "
                               f"different shapes: {sorted(shapes)}")
            break
    raise_together("restore planning", error)


@dataclass(frozen=True, slots=True)
class ModelInitialization:
    path: str
    destinations: tuple[str | None, ...]
    plural_destinations: bool
    source_model_key_prefix: str | None = None
    source_model_key_patterns: tuple[str, ...] = ()

    @property
    def coalescible(self) -> bool:
        return bool(self.destinations) and all(d is not None for d in self.destinations)

    def reads_same_source(self, other: "ModelInitialization") -> bool:
        return (self.path, self.source_model_key_prefix, self.source_model_key_patterns) == \
            (other.path, other.source_model_key_prefix, other.source_model_key_patterns)

    def load_kwargs(self) -> dict[str, Any]:
        out: dict[str, Any] = {"path": self.path,
                               "source_model_key_prefix": self.source_model_key_prefix}
        if self.source_model_key_patterns:
            out["source_model_key_patterns"] = self.source_model_key_patterns
        if self.plural_destinations:
            out["model_key_prefixes"] = self.destinations
        else:
            out["model_key_prefix"] = self.destinations[0]
        return out


def plan_model_initializations(entries: Mapping[str, Mapping[str, Any]], *, resume: bool,
                               ) -> tuple[ModelInitialization, ...]:
    """On resume only entries with ``resume_model_key_prefixes`` apply (frozen roles that
    checkpoints do not contain)."""
    plan: list[ModelInitialization] = []
    last = None
    for index, (label, entry) in enumerate(entries.items()):
        if resume:
            configured = entry.get("resume_model_key_prefixes")
            if not configured:
                continue
            destinations, plural = tuple(configured), True
        elif entry.get("model_key_prefixes") is not None:
            destinations, plural = tuple(entry["model_key_prefixes"]), True
        else:
            destinations, plural = (entry.get("model_key_prefix"),), False
        if entry.get("path") is None:
            warnings.warn(f"Skipping model initialization {label!r}: path is null.", stacklevel=2)
            continue
        item = ModelInitialization(
            path=entry["path"], destinations=destinations, plural_destinations=plural,
            source_model_key_prefix=entry.get("source_model_key_prefix"),
            source_model_key_patterns=tuple(entry.get("source_model_key_patterns", ())))
        if (plan and last == index - 1 and plan[-1].reads_same_source(item)
                and plan[-1].coalescible and item.coalescible):
            plan[-1] = replace(plan[-1], destinations=(*plan[-1].destinations, *item.destinations),
                               plural_destinations=True)
        else:
            plan.append(item)
        last = index
    return tuple(plan)
