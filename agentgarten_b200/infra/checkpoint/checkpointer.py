"""Distributed checkpointing on the torch DCP format.

Layout (one directory per save under ``save_dir``)::

    iter_%09d/tensor/            DCP directory (.metadata + *.distcp)
        model.<fqn>
        optimizers.<role>.state.<fqn>.{step,exp_avg,exp_avg_sq,master_param}
        optimizers.<role>.param_groups.<fqn>.<option>
        schedulers.<role>.{adapter,state.*}
        trainer.iteration, trainer.grad_scaler.*, trainer.rng_state.*
    iter_%09d/metadata.json      iteration, world size, runtime (mesh / CP topology)
    iter_%09d/dataloader/        per-rank loader cursors + their signature
    latest                       name of the newest complete checkpoint, written last

``async_mode="thread"`` snapshots device tensors to host memory synchronously and writes
the files in a background thread through a dedicated Gloo group; the ``latest`` pointer is
published only after every rank's write succeeded (checked collectively at ``finalize`` or
before the next save).  Loading is component-selective and partial: model weights can be
*overlaid* from another model's checkpoint or a HuggingFace safetensors directory under a
key prefix / regex mapping; optimizer and scheduler state restore progress but keep the
current recipe's options; the RNG state is validated at load and applied later, after the
data-loader workers have started.

Parity: reference ``wm/infra/checkpoint/checkpointer.py:99-1019``.
"""

from __future__ import annotations

import re
from collections.abc import Iterable, Mapping
from concurrent.futures import Future
from dataclasses import dataclass, field
from datetime import timedelta
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist

from agentgarten_b200.ops import kernel_status
from agentgarten_b200.infra.rng_state import (capture_distributed_rng_state,
                                              restore_distributed_rng_state,
                                              validate_distributed_rng_state)
from agentgarten_b200.utils import log
from agentgarten_b200.utils.io import atomic_put_text

from . import sidecar
from .common import gather_objects, raise_together, rank, warn_rank0, world_size
from .optimizer_state import load_optimizer_state, optimizer_state_for_save, optimizer_template
from .plan import (ModelRestorePlan, build_model_restore_plan, plan_model_initializations,
                   validate_overlay_target_shapes)
from .scheduler_state import (LAMBDA_LR_ADAPTER, restore_closed_form_scheduler_progress,
                              restore_grad_scaler_progress, restore_lambda_lr_progress,
                              scheduler_state_for_save)
from .source import LoadSource, component_fields, component_names, normalise_components

__all__ = ["DistributedCheckpointer", "LoadResult"]


@dataclass(frozen=True, slots=True)
class LoadResult:
    iteration: int = 0
    path: str | None = None
    loaded_components: tuple[str, ...] = ()
    missing_model_keys: tuple[str, ...] = ()
    unexpected_model_keys: tuple[str, ...] = ()
    loaded_model_keys: tuple[str, ...] = ()


@dataclass
class _Pending:
    name: str
    future: Future | None
    error: BaseException | None = None


def _unwrap(model: torch.nn.Module) -> torch.nn.Module:
    return getattr(model, "training_model", model)


def _flatten(tree: Mapping[str, Any], prefix: str = "") -> dict[str, Any]:
    out: dict[str, Any] = {}
    for key, value in tree.items():
        path = f"{prefix}{key}"
        if isinstance(value, Mapping):
            out.update(_flatten(value, path + "."))
        else:
            out[path] = value
    return out


def _nest(flat: Mapping[str, Any], prefix: str) -> dict[str, Any]:
    """Rebuild the nested dict below ``prefix`` from flat dotted keys (RNG state)."""
    out: dict[str, Any] = {}
    for key, value in flat.items():
        if not key.startswith(prefix):
            continue
        node = out
        *parents, leaf = key[len(prefix):].split(".")
        for part in parents:
            node = node.setdefault(part, {})
        node[leaf] = value
    return out


class DistributedCheckpointer:
    def __init__(self, save_dir: str | Path, *, async_mode: str | None = "disabled",
                 async_timeout_seconds: float = 3600.0) -> None:
        if async_mode not in (None, "none", "disabled", "thread"):
            raise ValueError(f"async_mode must be 'disabled' or 'thread', got {async_mode!r}")
        self.save_dir = Path(save_dir)
        self.latest_path = self.save_dir / "latest"
        self.async_mode = None if async_mode in (None, "none", "disabled") else async_mode
        self.async_timeout_seconds = float(async_timeout_seconds)
        self._pending: _Pending | None = None
        self._pending_rng: Mapping[str, Any] | None = None
        self._io_group = None
        if self.async_mode and dist.is_available() and dist.is_initialized():
            # file IO planning collectives must not share a communicator with model traffic
            self._io_group = dist.new_group(backend="gloo",
                                            timeout=timedelta(seconds=self.async_timeout_seconds))

    # ------------------------------------------------------------------- lifecycle
    def _publish_latest(self, name: str) -> None:
        error = None
        if rank() == 0:
            try:
                atomic_put_text(name + "\n", self.latest_path)
            except BaseException as e:
                error = e
        raise_together("latest pointer publication", error)

    def _wait(self, *, coordinate: bool = True) -> None:
        """Finish the pending save.  With ``coordinate`` all ranks agree on success and the
        ``latest`` pointer is published; without (error shutdown) nothing collective runs."""
        pending, self._pending = self._pending, None
        if pending is None:
            return
        error = pending.error
        if pending.future is not None and error is None:
            try:
                pending.future.result(timeout=self.async_timeout_seconds)
            except BaseException as e:
                error = e
        if not coordinate:
            if error is not None:
                log.warning(f"Pending checkpoint {pending.name} failed: {error}", rank0_only=False)
            return
        raise_together(f"write of {pending.name}", error)
        self._publish_latest(pending.name)

    def finalize(self) -> None:
        self._wait(coordinate=True)

    def finalize_after_error(self) -> None:
        self._wait(coordinate=False)

    # ------------------------------------------------------------------------ save
    def save(self, model: torch.nn.Module, optimizers: Mapping[str, Any],
             schedulers: Mapping[str, Any], grad_scaler: Any, *, iteration: int,
             dataloader: Any = None, runtime_metadata: Mapping[str, Any] | None = None) -> str:
        import torch.distributed.checkpoint as dcp

        self._wait(coordinate=True)
        root = _unwrap(model)
        # never write parameters that a timed-out kernel left incomplete (all ranks agree)
        some = next(iter(root.parameters()), None)
        if some is not None:
            kernel_status.raise_for_status(kernel_status.read(some.device), "checkpoint save")
        name = f"iter_{int(iteration):09d}"
        directory = self.save_dir / name
        rng = capture_distributed_rng_state()
        loader_snapshot = sidecar.capture_dataloader_snapshot(dataloader, runtime_metadata)
        model_state = root.checkpoint_model_state_dict(dict(root.state_dict()))
        state: dict[str, Any] = {
            "model": model_state,
            "optimizers": {role: optimizer_state_for_save(root, opt) for role, opt in optimizers.items()},
            "schedulers": {role: scheduler_state_for_save(s) for role, s in schedulers.items()},
            "trainer": {"iteration": int(iteration),
                        "grad_scaler": dict(grad_scaler.state_dict()) if grad_scaler is not None else {},
                        "rng_state": rng},
        }
        error = None
        if rank() == 0:
            try:
                (directory / "tensor").mkdir(parents=True, exist_ok=True)
            except BaseException as e:
                error = e
        raise_together("checkpoint directory creation", error)
        sidecar.save_checkpoint_metadata(directory, iteration=iteration, runtime_metadata=runtime_metadata)
        sidecar.save_dataloader_snapshot(directory, loader_snapshot)
        writer = dcp.FileSystemWriter(str(directory / "tensor"))
        if self.async_mode == "thread":
            try:
                future = dcp.async_save(state, storage_writer=writer, process_group=self._io_group)
                self._pending = _Pending(name, future)
            except BaseException as e:
                self._pending = _Pending(name, None, e)
        else:
            try:
                dcp.save(state, storage_writer=writer)
                self._pending = _Pending(name, None)
            except BaseException as e:
                self._pending = _Pending(name, None, e)
            self._wait(coordinate=True)
        restore_distributed_rng_state(rng)  # saving must not move the training streams
        return str(directory)

    # --------------------------------------------------------------- initial weights
    def initialize_model(self, model: torch.nn.Module, initializations: Mapping[str, Any] | None,
                         *, resume: bool = False) -> None:
        """Apply the ``train.model_initializations`` overlays in order."""
        for item in plan_model_initializations(dict(initializations or {}), resume=resume):
            self.load(model, {}, {}, None, components=("model",), **item.load_kwargs())

    # ------------------------------------------------------------------------ load
    def _resolve(self, path: str | Path | None) -> Path | None:
        """``None`` loads nothing; the literal ``"latest"`` follows ``save_dir/latest`` (a missing
        or empty pointer is an error; an absolute target is taken as it is, a relative one is
        under ``save_dir``); anything else names the checkpoint directory itself."""
        if path is None:
            return None
        if str(path) != "latest":
            return Path(path)
        pointer = self.latest_path
        if not pointer.is_file():
            raise FileNotFoundError(f"No latest checkpoint pointer at {pointer}")
        target = pointer.read_text().strip()
        if not target:
            raise FileNotFoundError(f"Latest checkpoint pointer is empty: {pointer}")
        target_path = Path(target)
        return target_path if target_path.is_absolute() else self.save_dir / target_path

    def load(self, model: torch.nn.Module, optimizers: Mapping[str, Any] | None = None,
             schedulers: Mapping[str, Any] | None = None, grad_scaler: Any = None, *,
             path: str | Path | None = "latest", components: Iterable[str] | None = None,
             dataloader: Any = None, runtime_metadata: Mapping[str, Any] | None = None,
             model_key_prefix: str | None = None,
             model_key_prefixes: Iterable[str | None] | None = None,
             source_model_key_prefix: str | None = None,
             source_model_key_patterns: Iterable[str] | None = None) -> LoadResult:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint import DefaultLoadPlanner

        source_model_key_patterns = tuple(source_model_key_patterns or ())
        decision: list[Any] = [None, None]
        if rank() == 0:
            try:
                found = self._resolve(path)
                decision = [None if found is None else str(found), None]
            except FileNotFoundError as error:
                decision = [None, str(error)]
        if world_size() > 1:
            dist.broadcast_object_list(decision, src=0)
        if decision[1] is not None:  # every rank fails together
            raise FileNotFoundError(decision[1])
        if decision[0] is None:
            return LoadResult()
        directory = Path(decision[0])
        root = _unwrap(model)
        optimizers, schedulers = dict(optimizers or {}), dict(schedulers or {})
        selected = normalise_components(components, include_dataloader=dataloader is not None)
        overlay = (model_key_prefix is not None or model_key_prefixes is not None
                   or source_model_key_prefix is not None or bool(tuple(source_model_key_patterns)))
        source = LoadSource.open(directory, source_model_key_prefix if overlay else None)
        template: dict[str, Any] = {}
        loaded: list[str] = []

        # ---- model
        plan: ModelRestorePlan | None = None
        live_state = root.checkpoint_model_state_dict(dict(root.state_dict())) if not overlay \
            else dict(root.state_dict())
        head = "" if source.flat_model else "model."
        if source.has("model", selected):
            saved_model_keys = [k[len(head):] for k in source.state_keys if k.startswith(head)]
            destinations = tuple(model_key_prefixes) if model_key_prefixes is not None \
                else (model_key_prefix,)
            plan = build_model_restore_plan(
                live_keys=live_state.keys(), saved_keys=saved_model_keys, overlay=overlay,
                source_prefix=source_model_key_prefix, destination_prefixes=destinations,
                source_patterns=[re.compile(p) for p in source_model_key_patterns])
            if overlay:
                validate_overlay_target_shapes(plan, live_state)
            for entry in plan.entries:
                template[head + entry.source_key] = live_state[entry.template_key]
            loaded.append("model")

        # ---- optimizers / schedulers / trainer
        opt_fields: dict[str, set[str]] = {}
        if source.has("optimizers", selected):
            saved_roles = component_names(source.state_keys, "optimizers")
            for role, opt in optimizers.items():
                if role not in saved_roles:
                    warn_rank0(f"Checkpoint has no optimizer state for role '{role}'; keeping it fresh.")
                    continue
                fields = component_fields(source.state_keys, "optimizers", role)
                opt_fields[role] = fields
                for k, v in optimizer_template(root, opt, fields).items():
                    template[f"optimizers.{role}.{k}"] = v
            loaded.append("optimizers")
        sched_fields: dict[str, set[str]] = {}
        if source.has("schedulers", selected):
            saved_roles = component_names(source.state_keys, "schedulers")
            for role in schedulers:
                if role in saved_roles:
                    sched_fields[role] = component_fields(source.state_keys, "schedulers", role)
            loaded.append("schedulers")
        trainer_fields = component_fields(source.state_keys, "trainer") \
            if source.has("trainer", selected) else set()
        if trainer_fields:
            loaded.append("trainer")

        # One collective read for the tensors; small objects are read by every rank.
        object_keys = [f"schedulers.{r}.{f}" for r, fs in sched_fields.items() for f in fs]
        object_keys += [f"trainer.{f}" for f in trainer_fields]
        object_keys += [f"optimizers.{r}.{f}" for r, fs in opt_fields.items() for f in fs
                        if f.startswith("param_groups.") or f.endswith(".step")]
        error = None
        try:
            self._read(dcp, DefaultLoadPlanner, source, template, object_keys)
        except BaseException as e:
            error = e
        raise_together("tensor read", error)
        objects = self._objects

        # ---- apply
        missing: tuple[str, ...] = ()
        unexpected: tuple[str, ...] = ()
        restored: tuple[str, ...] = ()
        if plan is not None:
            restored = tuple(target for entry in plan.entries for target in entry.targets)
            with torch.no_grad():
                for entry in plan.entries:
                    value = template[head + entry.source_key]
                    for target in entry.targets[1:]:
                        live_state[target].copy_(value)
            missing, unexpected = plan.missing_model_keys, plan.unexpected_model_keys
            if missing or unexpected:
                warn_rank0(f"Model restore from {directory}: {len(missing)} missing, "
                           f"{len(unexpected)} unexpected keys"
                           + (f" (missing e.g. {missing[:3]})" if missing else ""))
            for opt in (getattr(root, "optimizer_dict", None) or {}).values():
                engine = getattr(opt, "engine", None)
                if engine is not None and "optimizers" not in loaded:
                    engine.refresh_master()  # new bf16 weights => new FP32 master copies
        for role, fields in opt_fields.items():
            prefix = f"optimizers.{role}."
            values = {k[len(prefix):]: v for k, v in {**template, **objects}.items()
                      if k.startswith(prefix)}
            load_optimizer_state(role, root, optimizers[role], values)
        for role, fields in sched_fields.items():
            prefix = f"schedulers.{role}.state."
            state = {k[len(prefix):]: v for k, v in objects.items() if k.startswith(prefix)}
            scheduler = schedulers[role]
            adapter = objects.get(f"schedulers.{role}.adapter")
            if adapter == LAMBDA_LR_ADAPTER and isinstance(scheduler, torch.optim.lr_scheduler.LambdaLR):
                restore_lambda_lr_progress(scheduler, state, set(state))
            else:
                restore_closed_form_scheduler_progress(role, scheduler, state, set(state))
        iteration = 0
        if trainer_fields:
            iteration = int(objects.get("trainer.iteration", 0))
            if grad_scaler is not None:
                saved = {k[len("trainer.grad_scaler."):]: v for k, v in objects.items()
                         if k.startswith("trainer.grad_scaler.")}
                restore_grad_scaler_progress(grad_scaler, dict(grad_scaler.state_dict()), saved, set(saved))
            rng = _nest(objects, "trainer.rng_state.")
            if rng:
                try:
                    validate_distributed_rng_state(rng)
                    self._pending_rng = rng
                except RuntimeError as e:
                    warn_rank0(f"Not restoring RNG state: {e}")
        if "dataloader" in selected and dataloader is not None:
            sidecar.warn_runtime_metadata_changes(directory, runtime_metadata)
            if sidecar.restore_dataloader_snapshot(directory, dataloader, runtime_metadata):
                loaded.append("dataloader")
        return LoadResult(iteration, str(directory), tuple(loaded), missing, unexpected, restored)

    def _read(self, dcp, planner_type, source: LoadSource, template: dict[str, Any],
              object_keys: list[str]) -> None:
        """Tensors go through one DCP load into the live storage; non-tensor entries
        (ints, floats, strings, small CPU tensors) are read into ``self._objects``."""
        self._objects: dict[str, Any] = {}
        meta = source.metadata.state_dict_metadata
        request = dict(template)
        for key in object_keys:
            if key in request or key not in meta:
                continue
            entry = meta[key]
            if hasattr(entry, "size") and hasattr(entry, "properties"):
                request[key] = torch.empty(tuple(entry.size), dtype=entry.properties.dtype)
            else:
                request[key] = None
        if not request:
            return
        tensors = {k: v for k, v in request.items() if v is not None}
        blobs = {k: None for k, v in request.items() if v is None}
        payload = {**tensors, **blobs}
        dcp.load(payload, storage_reader=source.reader,
                 planner=planner_type(allow_partial_load=True))
        for key in object_keys:
            if key in payload and key not in template:
                self._objects[key] = payload[key]

    def restore_pending_rng_state(self) -> bool:
        rng, self._pending_rng = self._pending_rng, None
        if rng is None:
            return False
        restore_distributed_rng_state(rng)
        return True
