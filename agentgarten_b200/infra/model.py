"""Base class of training objectives.

A ``Model`` owns named optimizers/schedulers ("roles"), chooses which roles are active in
an iteration, yields the loss closures of a step, and filters what goes to checkpoints.

Parity: reference ``wm/infra/model.py:40-339``.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from collections.abc import Callable, Iterator, Mapping, Sequence
from dataclasses import dataclass
from typing import Any, Protocol, TypeAlias, runtime_checkable

import torch
import torch.distributed as dist

from .config import instantiate
from .parameter_groups import enable_only, group_by_declarations, split_matrices_from_vectors

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


def _ranks_sharing_a_clip(mesh) -> tuple[int, ...]:
    """Global ranks of a context-parallel mesh; a missing or trivial mesh is this rank alone."""
    if mesh is not None and mesh.size() > 1:
        return tuple(dist.get_process_group_ranks(mesh.get_group()))
    return (dist.get_rank(),) if dist.is_available() and dist.is_initialized() else (0,)


class ContextParallelContext:
    """This rank's place in its context-parallel group.

    Without context parallelism every rank is a group of its own (``size`` 1, leader of
    itself).  With it, ``groups`` lists every group of the job in sorted order and
    ``artifact_rank`` is the index of this rank's group in that list, so that one writer per
    group (its leader) names sample files.
    """

    def __init__(self, mesh=None) -> None:
        members = _ranks_sharing_a_clip(mesh)
        self.mesh = mesh
        self.size = len(members)
        self.leader_global_rank = members[0]
        if self.size == 1:
            self.group, self.rank, self.groups = None, 0, ()
            self.artifact_rank = members[0]
            return
        self.group = mesh.get_group()
        self.rank = int(mesh.get_local_rank())
        reported: list[Any] = [None] * dist.get_world_size()
        dist.all_gather_object(reported, members)
        self.groups = tuple(sorted(set(filter(None, reported))))
        self.artifact_rank = self.groups.index(members)

    @property
    def enabled(self) -> bool:
        return self.size > 1

    @property
    def is_leader(self) -> bool:
        return self.rank == 0

    def global_rank(self, local_rank: int) -> int:
        if self.enabled:
            return dist.get_global_rank(self.group, int(local_rank))
        return self.leader_global_rank

    def broadcast_objects(self, values: list[Any], *, source_rank: int) -> None:
        """In-place broadcast inside the group (a no-op for a group of one)."""
        if self.enabled:
            dist.broadcast_object_list(values, src=self.global_rank(source_rank), group=self.group)

    def checkpoint_topology(self) -> dict[str, Any] | None:
        if not self.enabled:
            return None
        return {"size": self.size, "groups": [list(members) for members in self.groups]}


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
        """All networks of one objective must split clips over the same ranks."""
        mine = _ranks_sharing_a_clip(mesh)
        for other in role_meshes:
            if _ranks_sharing_a_clip(other) != mine:
                raise ValueError("all Networks in one training objective must use the same "
                                 "context-parallel topology")
        self._context_parallel_context = ContextParallelContext(mesh)

    # ------------------------------------------------------------ parameter groups
    _group_module_trainable_parameters = staticmethod(group_by_declarations)

    def _group_trainable_parameters(self) -> list[dict[str, Any]]:
        groups = group_by_declarations(self, self.optimizer_parameter_groups)
        if self.optimizer_split_decay_groups and not self.optimizer_parameter_groups:
            groups = split_matrices_from_vectors(groups)
        return groups

    def configure_trainable_parameters(self, patterns: str | Sequence[str] | None, *,
                                       module: torch.nn.Module | None = None) -> None:
        """``None`` leaves everything as it is; otherwise only matching parameters train."""
        if patterns is not None:
            enable_only(self if module is None else module, patterns)

    # ------------------------------------------------------------------ optimizers
    def init_optimizer_scheduler(self, optimizer_config, scheduler_config):
        optimizer = instantiate(optimizer_config, params=self._group_trainable_parameters())
        self.optimizer_dict = {"net": optimizer}
        self.scheduler_dict = {"net": instantiate(scheduler_config, optimizer=optimizer)}
        return self.optimizer_dict, self.scheduler_dict

    def get_optimizer_names(self, iteration: int) -> tuple[str, ...]:
        return ("net",)

    def _binding(self, name: str) -> OptimizerBinding:
        optimizer, scheduler = self.optimizer_dict.get(name), self.scheduler_dict.get(name)
        if optimizer is None or scheduler is None:
            raise RuntimeError(f"Optimizer role {name!r} is not registered with a scheduler")
        if getattr(scheduler, "optimizer", None) is not optimizer:
            raise RuntimeError(f"Scheduler for role {name!r} owns a different optimizer")
        return OptimizerBinding(name, optimizer, scheduler)

    def get_optimizer_bindings(self, iteration: int) -> tuple[OptimizerBinding, ...]:
        """The (name, optimizer, scheduler) triples that take part in ``iteration``."""
        names = tuple(self.get_optimizer_names(iteration))
        if not names:
            raise RuntimeError("Model selected no optimizer for this iteration")
        if len(names) != len(set(names)):
            raise RuntimeError(f"Optimizer roles are selected more than once: {names}")
        bindings = tuple(self._binding(name) for name in names)
        # roles stepped in one update must own disjoint parameters (each would be unscaled and
        # stepped twice otherwise); roles that are idle this iteration may share them
        held_by: dict[int, str] = {}
        for binding in bindings:
            for group in binding.optimizer.param_groups:
                for parameter in group["params"]:
                    holder = held_by.setdefault(id(parameter), binding.name)
                    if holder != binding.name:
                        raise RuntimeError(
                            f"Active optimizer roles {holder!r} and {binding.name!r} share a "
                            "parameter; active roles must own disjoint parameters")
        return bindings

    def is_cadence_due(self, iteration: int, interval: int | None) -> bool:
        if interval is None or int(interval) <= 0:
            return False
        return int(iteration) > 0 and int(iteration) % int(interval) == 0

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
