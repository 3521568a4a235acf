"""Base class of training objectives.

A ``Model`` owns named optimizers/schedulers ("roles"), chooses which roles are active in
an iteration, yields the loss closures of a step, and filters what goes to checkpoints.

Parity: reference ``wm/infra/model.py:40-339``.
"""

from __future__ import annotations

import re
from abc import ABC, abstractmethod
from collections.abc import Callable, Iterator, Mapping, Sequence
from dataclasses import dataclass
from typing import Any, Protocol, TypeAlias, runtime_checkable

import torch
import torch.distributed as dist

from .config import instantiate

StepOutput: TypeAlias = tuple[dict[str, Any], torch.Tensor]
TrainingClosure: TypeAlias = Callable[[], StepOutput]
TrainingClosureSpec: TypeAlias = tuple[str, TrainingClosure, bool]

__all__ = [
    "ContextParallelContext",
    "LifecycleCadence",
    "Model",
    "OptimizerBinding",
    "StepOutput",
    "TrainingClosure",
    "TrainingClosureSpec",
]


@runtime_checkable
class LifecycleCadence(Protocol):
    def is_cadence_due(self, iteration: int, interval: int | None) -> bool: ...


@dataclass(frozen=True, slots=True)
class OptimizerBinding:
    name: str
    optimizer: torch.optim.Optimizer
    scheduler: Any


def _mesh_ranks(mesh) -> tuple[int, ...]:
    if mesh is None or mesh.size() <= 1:
        if dist.is_available() and dist.is_initialized():
            return (dist.get_rank(),)
        return (0,)
    return tuple(dist.get_process_group_ranks(mesh.get_group()))


class ContextParallelContext:
    """Where this rank sits in its context-parallel group (if any).

    ``artifact_rank`` numbers the CP groups, so one writer per group produces sample files.
    """

    def __init__(self, mesh=None) -> None:
        self.mesh = mesh
        self.group = None
        self.size, self.rank = 1, 0
        self.groups: tuple[tuple[int, ...], ...] = ()
        me = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        self.leader_global_rank = me
        self.artifact_rank = me
        if mesh is None or mesh.size() <= 1:
            return
        self.group = mesh.get_group()
        self.size = int(mesh.size())
        self.rank = int(mesh.get_local_rank())
        mine = tuple(dist.get_process_group_ranks(self.group))
        self.leader_global_rank = mine[0]
        everyone: list[Any] = [None] * dist.get_world_size()
        dist.all_gather_object(everyone, mine)
        self.groups = tuple(sorted({g for g in everyone if g is not None}))
        self.artifact_rank = self.groups.index(mine)

    @property
    def enabled(self) -> bool:
        return self.size > 1

    @property
    def is_leader(self) -> bool:
        return self.rank == 0

    def global_rank(self, local_rank: int) -> int:
        if not self.enabled:
            return self.leader_global_rank
        return dist.get_global_rank(self.group, int(local_rank))

    def broadcast_objects(self, values: list[Any], *, source_rank: int) -> None:
        if self.enabled:
            dist.broadcast_object_list(values, src=self.global_rank(source_rank), group=self.group)

    def checkpoint_topology(self) -> dict[str, Any] | None:
        if not self.enabled:
            return None
        return {"size": self.size, "groups": [list(g) for g in self.groups]}


class Model(torch.nn.Module, ABC):
    def __init__(self, optimizer_parameter_groups: Sequence[Mapping[str, Any]] | None = None,
                 optimizer_split_decay_groups: bool = False) -> None:
        super().__init__()
        self.optimizer_parameter_groups = optimizer_parameter_groups
        self.optimizer_split_decay_groups = bool(optimizer_split_decay_groups)
        self.optimizer_dict: dict[str, torch.optim.Optimizer] = {}
        self.scheduler_dict: dict[str, Any] = {}
        self._context_parallel_context = ContextParallelContext()

    # ------------------------------------------------------------ context parallel
    @property
    def context_parallel_context(self) -> ContextParallelContext:
        return self._context_parallel_context

    def register_context_parallel_mesh(self, mesh, *role_meshes) -> None:
        expected = _mesh_ranks(mesh)
        if any(_mesh_ranks(other) != expected for other in role_meshes):
            raise ValueError("all Networks in one training objective must use the same "
                             "context-parallel topology")
        self._context_parallel_context = ContextParallelContext(mesh)

    # ------------------------------------------------------------ parameter groups
    @staticmethod
    def _group_module_trainable_parameters(module: torch.nn.Module,
                                           declarations: Sequence[Mapping[str, Any]] | None = None,
                                           ) -> list[dict[str, Any]]:
        """Split trainable parameters into optimizer groups by regex declarations.

        A declaration is ``{"patterns": [...], **group options}``; a parameter joins the
        first declaration one of whose patterns fully matches any of its names (shared
        parameters have several).  Unmatched parameters form the leading default group.
        """
        live = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        if not declarations:
            return [{"params": [p for _, p in live]}]
        aliases: dict[int, list[str]] = {id(p): [] for _, p in live}
        for name, p in module.named_parameters(remove_duplicate=False):
            if id(p) in aliases:
                aliases[id(p)].append(name)
        taken: set[int] = set()
        declared: list[dict[str, Any]] = []
        for declaration in declarations:
            patterns = declaration["patterns"]
            patterns = (patterns,) if isinstance(patterns, str) else tuple(patterns)
            compiled = [re.compile(p) for p in patterns]
            chosen = [p for _, p in live if id(p) not in taken and any(
                c.fullmatch(alias) for c in compiled for alias in aliases[id(p)])]
            if not chosen:
                continue
            taken.update(id(p) for p in chosen)
            declared.append({**{k: v for k, v in declaration.items() if k != "patterns"},
                             "params": chosen})
        rest = [p for _, p in live if id(p) not in taken]
        return ([{"params": rest}] if rest else []) + declared

    def _group_trainable_parameters(self) -> list[dict[str, Any]]:
        groups = self._group_module_trainable_parameters(self, self.optimizer_parameter_groups)
        if not self.optimizer_split_decay_groups or self.optimizer_parameter_groups:
            return groups
        out: list[dict[str, Any]] = []
        for group in groups:
            options = {k: v for k, v in group.items() if k != "params"}
            matrices = [p for p in group["params"] if p.ndim >= 2]
            vectors = [p for p in group["params"] if p.ndim < 2]
            out.extend({**options, "params": sel} for sel in (matrices, vectors) if sel)
        return out

    def configure_trainable_parameters(self, patterns: str | Sequence[str] | None, *,
                                       module: torch.nn.Module | None = None) -> None:
        """Freeze everything, then re-enable parameters whose (any) name fully matches."""
        if patterns is None:
            return
        patterns = (patterns,) if isinstance(patterns, str) else tuple(patterns)
        compiled = [re.compile(p) for p in patterns]
        target = self if module is None else module
        target.requires_grad_(False)
        for name, parameter in target.named_parameters(remove_duplicate=False):
            if any(c.fullmatch(name) for c in compiled):
                parameter.requires_grad_(True)

    # ------------------------------------------------------------------ optimizers
    def init_optimizer_scheduler(self, optimizer_config, scheduler_config):
        optimizer = instantiate(optimizer_config, params=self._group_trainable_parameters())
        scheduler = instantiate(scheduler_config, optimizer=optimizer)
        self.optimizer_dict = {"net": optimizer}
        self.scheduler_dict = {"net": scheduler}
        return self.optimizer_dict, self.scheduler_dict

    def get_optimizer_names(self, iteration: int) -> tuple[str, ...]:
        del iteration
        return ("net",)

    def get_optimizer_bindings(self, iteration: int) -> tuple[OptimizerBinding, ...]:
        names = tuple(self.get_optimizer_names(iteration))
        if not names:
            raise RuntimeError("Model selected no optimizer for this iteration")
        if len(set(names)) != len(names):
            raise RuntimeError(f"Optimizer roles are selected more than once: {names}")
        bindings = []
        for name in names:
            optimizer, scheduler = self.optimizer_dict.get(name), self.scheduler_dict.get(name)
            if optimizer is None or scheduler is None:
                raise RuntimeError(f"Optimizer role {name!r} is not registered with a scheduler")
            if getattr(scheduler, "optimizer", None) is not optimizer:
                raise RuntimeError(f"Scheduler for role {name!r} owns a different optimizer")
            bindings.append(OptimizerBinding(name, optimizer, scheduler))
        if len(bindings) > 1:
            # Roles stepped together must own disjoint parameters.
            owner: dict[int, str] = {}
            for binding in bindings:
                for group in binding.optimizer.param_groups:
                    for p in group["params"]:
                        before = owner.setdefault(id(p), binding.name)
                        if before != binding.name:
                            raise RuntimeError(
                                f"Active optimizer roles {before!r} and {binding.name!r} share a "
                                "parameter; active roles must own disjoint parameters")
        return tuple(bindings)

    def is_cadence_due(self, iteration: int, interval: int | None) -> bool:
        return (interval is not None and int(interval) > 0 and int(iteration) > 0
                and int(iteration) % int(interval) == 0)

    # ------------------------------------------------------------------- lifecycle
    def parallelize(self, device) -> None:
        self.to(device)

    def prepare_data_batch(self, data_batch: dict[str, Any]) -> dict[str, Any]:
        return data_batch

    def training_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        raise NotImplementedError

    def training_step_closures(self, data_batch: dict[str, Any], iteration: int,
                               ) -> Iterator[TrainingClosureSpec]:
        yield "train", lambda: self.training_step(data_batch, iteration), True

    @torch.no_grad()
    def validation_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        raise NotImplementedError

    @torch.inference_mode()
    @abstractmethod
    def sample(self, data_batch: dict[str, Any], **sampling_options: Any) -> Any:
        raise NotImplementedError

    def checkpoint_model_state_dict(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        return state_dict
