"""Flattened optimizer state: ``state.<fqn>.<slot>`` and ``param_groups.<fqn>.<option>``.

Rules on restore: a parameter that had no state in the checkpoint gets none created; the
parameter-group options of the *current* recipe (learning rate, betas, ...) win over the
saved ones, with a warning when they differ.  With the sharded CUDA optimizer every rank
saves its own dim-0 chunk of ``exp_avg`` / ``exp_avg_sq`` / ``master_param`` as a
``Shard(0)`` DTensor, which is the layout an FSDP2 run produces for the same parameter.

Parity: reference ``wm/infra/checkpoint/optimizer_state.py:32-260``.
"""

from __future__ import annotations

import copy
from collections.abc import Mapping
from typing import Any

import torch
import torch.distributed as dist

from .common import warn_rank0

__all__ = ["load_optimizer_state", "optimizer_group_options", "optimizer_options_differ",
           "optimizer_state_for_save", "optimizer_template", "option_equal"]

_SLOTS = ("exp_avg", "exp_avg_sq", "master_param")


def option_equal(left: Any, right: Any) -> bool:
    if isinstance(left, torch.Tensor) or isinstance(right, torch.Tensor):
        return isinstance(left, torch.Tensor) and isinstance(right, torch.Tensor) \
            and left.shape == right.shape and bool(torch.equal(left, right))
    if isinstance(left, (list, tuple)) and isinstance(right, (list, tuple)):
        return len(left) == len(right) and all(option_equal(a, b) for a, b in zip(left, right))
    try:
        return bool(left == right)
    except (TypeError, ValueError):
        return left is right


def _snapshot(value: Any) -> Any:
    if isinstance(value, torch.Tensor):
        return value.detach().clone()
    if isinstance(value, Mapping):
        return {k: _snapshot(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_snapshot(v) for v in value)
    return copy.deepcopy(value)


def optimizer_group_options(optimizer) -> tuple[dict[str, Any], ...]:
    return tuple({k: _snapshot(v) for k, v in g.items() if k != "params"}
                 for g in optimizer.param_groups)


def _names(model: torch.nn.Module) -> dict[int, str]:
    return {id(p): n for n, p in model.named_parameters()}


def _shard_mesh(optimizer):
    """Device mesh of the engine's shard group, for wrapping state chunks as DTensors.

    One node: the 1-D mesh over the shard group's ranks.  Several nodes (state sharded inside
    a node and replicated across nodes): the 2-D ``(replicate, shard)`` mesh over all ranks,
    so every rank is inside the mesh and each replica's chunks are saved and restored."""
    engine = getattr(optimizer, "engine", None)
    if engine is None or engine.world == 1:
        return None
    if not hasattr(engine, "_dcp_mesh"):
        import torch.distributed as dist
        from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

        if getattr(engine, "replica_group", None) is not None:
            replicas = dist.get_world_size() // engine.world
            engine._dcp_mesh = init_device_mesh(engine.device.type, (replicas, engine.world),
                                                mesh_dim_names=("replicate", "shard"))
        else:
            ranks = dist.get_process_group_ranks(engine.group) if engine.group is not None \
                else list(range(engine.world))
            if ranks == list(range(dist.get_world_size())):
                engine._dcp_mesh = init_device_mesh(engine.device.type, (engine.world,),
                                                    mesh_dim_names=("shard",))
            else:
                engine._dcp_mesh = DeviceMesh(engine.device.type, ranks, mesh_dim_names=("shard",))
    return engine._dcp_mesh


def _as_saved(optimizer, p: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """Wrap this rank's chunk of a state tensor as a Shard(0) DTensor (multi-rank engine).
    Zero-dimensional parameters cannot be sharded: their state is saved as a plain tensor
    (it lives on the first rank of the shard group and is empty elsewhere)."""
    mesh = _shard_mesh(optimizer)
    info = optimizer.engine.info[id(p)] if mesh is not None else None
    if mesh is None or len(info.global_shape) == 0:
        return value
    from torch.distributed.tensor import DTensor, Replicate, Shard

    shape = torch.Size(info.global_shape)
    stride = torch.empty(shape, device="meta").stride()
    placements = (Shard(0),) if mesh.ndim == 1 else (Replicate(), Shard(0))
    return DTensor.from_local(value, mesh, placements, run_check=False, shape=shape, stride=stride)


def optimizer_state_for_save(model: torch.nn.Module, optimizer) -> dict[str, Any]:
    engine = getattr(optimizer, "engine", None)
    if engine is not None:
        engine.publish_state()
    names = _names(model)
    out: dict[str, Any] = {}
    for group in optimizer.param_groups:
        options = {k: v for k, v in group.items() if k != "params"}
        for p in group["params"]:
            fqn = names.get(id(p))
            if fqn is None:
                continue
            for key, value in options.items():
                out[f"param_groups.{fqn}.{key}"] = list(value) if isinstance(value, tuple) else value
            state = optimizer.state.get(p)
            if not state:
                continue
            for slot, value in state.items():
                if isinstance(value, torch.Tensor) and slot in _SLOTS:
                    value = _as_saved(optimizer, p, value)
                elif isinstance(value, torch.Tensor) and value.ndim == 0:
                    value = value.detach().cpu().clone()
                out[f"state.{fqn}.{slot}"] = value
    return out


def optimizer_template(model: torch.nn.Module, optimizer, saved_fields: set[str]) -> dict[str, Any]:
    """Load targets for exactly the fields the checkpoint has (never more)."""
    engine = getattr(optimizer, "engine", None)
    if engine is not None:
        engine.publish_state()
    names = _names(model)
    template: dict[str, Any] = {}
    for group in optimizer.param_groups:
        betas = group.get("betas", (0.9, 0.999))
        for p in group["params"]:
            fqn = names.get(id(p))
            if fqn is None:
                continue
            for field in saved_fields:
                prefix = f"state.{fqn}."
                if not field.startswith(prefix):
                    continue
                slot = field[len(prefix):]
                if slot == "step":
                    template[field] = torch.zeros((), dtype=torch.float32)
                elif slot in _SLOTS:
                    if (slot == "exp_avg" and float(betas[0]) == 0) or \
                            (slot == "exp_avg_sq" and float(betas[1]) == 0):
                        continue
                    have = optimizer.state.get(p, {}).get(slot)
                    if engine is not None:
                        target = _as_saved(optimizer, p, have)
                    else:
                        target = have if isinstance(have, torch.Tensor) else \
                            torch.zeros_like(p, dtype=torch.float32)
                    template[field] = target
    for field in saved_fields:
        if field.startswith("param_groups."):
            template[field] = None  # non-tensor entries are read as objects
    return {k: v for k, v in template.items() if v is not None}


def optimizer_options_differ(left: Mapping[str, Any], right: Mapping[str, Any]) -> bool:
    if set(left) != set(right):
        return True
    for key in left:
        head, dot, field = key.rpartition(".")
        if dot and field == "lr" and f"{head}.initial_lr" in left and f"{head}.initial_lr" in right:
            continue  # schedulers move lr; the configured base is compared via initial_lr
        if not option_equal(left[key], right[key]):
            return True
    return False


def load_optimizer_state(name: str, model: torch.nn.Module, optimizer, loaded: Mapping[str, Any]) -> None:
    names = _names(model)
    engine = getattr(optimizer, "engine", None)
    touched = False
    for group in optimizer.param_groups:
        for p in group["params"]:
            fqn = names.get(id(p))
            if fqn is None:
                continue
            prefix = f"state.{fqn}."
            fields = {k[len(prefix):]: v for k, v in loaded.items() if k.startswith(prefix)}
            if not fields:
                continue
            state = optimizer.state[p]
            for slot, value in fields.items():
                if hasattr(value, "to_local"):
                    value = value.to_local()
                if slot == "step":
                    state["step"] = torch.as_tensor(float(value), dtype=torch.float32)
                elif isinstance(value, torch.Tensor):
                    state[slot] = value.detach().to(device=p.device, dtype=torch.float32)
            touched = True
    if engine is not None and touched:
        engine.adopt_state()
    saved_options = {k: v for k, v in loaded.items() if k.startswith("param_groups.")}
    if saved_options:
        current = {k: v for k, v in optimizer_state_for_save(model, optimizer).items()
                   if k.startswith("param_groups.") and k in saved_options}
        if optimizer_options_differ(saved_options, current):
            warn_rank0(f"Optimizer '{name}' resumed its state while keeping current "
                       "parameter-group options.")
