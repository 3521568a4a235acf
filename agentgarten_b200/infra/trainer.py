"""Update-counted training loop.

One *iteration* is one optimizer update; it consumes ``grad_accum_steps`` microbatches, and
each microbatch may run several loss closures (e.g. fake-score + discriminator).  Per
update: gradients are combined across ranks (the sharded engine does this in its
reduce-scatter kernel, DDP in its reducer), callbacks may clip, all ranks agree on whether
the gradients are finite, the active optimizers and schedulers step (or the step is
skipped everywhere), gradients are cleared.  Checkpoint and validation cadence are asked of
the model, which may count something other than raw iterations.

Exact resume: state is restored first, the loader's workers are started next, and only then
is the checkpointed RNG put back, so worker start-up cannot shift the random streams.
Validation runs with the training mode, loader cursor and RNG streams preserved.

Parity: reference ``wm/infra/trainer.py:43-627``.
"""

from __future__ import annotations

import warnings
from collections.abc import Callable, Iterable, Iterator, Mapping
from contextlib import contextmanager
from copy import deepcopy
from dataclasses import dataclass
from functools import partial
from pathlib import Path
from typing import Any

import torch

from agentgarten_b200.utils.misc import preserve_training_mode, to

from .batch_transport import fetch_batch, prepare_batch
from .callbacks.base import CallbackGroup
from .distributed import DistributedDataParallel, ddp_sync_grad, is_rank0
from .model import Model
from agentgarten_b200.utils.trace import span

from agentgarten_b200.parallel import zero

from .nonfinite import synchronize_found_nonfinite
from .rng_state import isolated_rng

__all__ = ["Trainer", "TrainingStepResult"]

Batch = dict[str, Any]


@dataclass(frozen=True, slots=True)
class TrainingStepResult:
    output_batch: Batch
    loss: torch.Tensor
    grad_accum_step: int
    did_update: bool
    found_nonfinite: bool = False


class _NoScaler:
    """Stand-in for a disabled ``torch.amp.GradScaler``."""

    def is_enabled(self) -> bool:
        return False

    def scale(self, loss):
        return loss

    def unscale_(self, optimizer) -> None:
        return

    def step(self, optimizer):
        return optimizer.step()

    def update(self) -> None:
        return

    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, state) -> None:
        return


@contextmanager
def _keep_loader_cursor(loader) -> Iterator[None]:
    get, put = getattr(loader, "state_dict", None), getattr(loader, "load_state_dict", None)
    saved = deepcopy(get()) if callable(get) and callable(put) else None
    try:
        yield
    finally:
        if saved is not None:
            put(saved)


def _pick(registry: Mapping[str, Any], names, *, label: str) -> dict[str, Any]:
    if names is None:
        return dict(registry)
    wanted = (names,) if isinstance(names, str) else tuple(names)
    wanted = tuple(dict.fromkeys(str(n) for n in wanted))
    unknown = [n for n in wanted if n not in registry]
    if unknown:
        raise ValueError(f"Unknown checkpoint {label} name(s): {', '.join(unknown)}; "
                         f"available: {', '.join(sorted(registry)) or '<none>'}")
    return {n: registry[n] for n in wanted}


def _root(model: torch.nn.Module) -> Model:
    if isinstance(model, DistributedDataParallel):
        return model.training_model
    if isinstance(model, torch.nn.parallel.DistributedDataParallel):
        raise TypeError("Trainer closures cannot run through stock PyTorch DDP; use "
                        "wrap_ddp(), whose forward_closure() enters the reducer lifecycle.")
    if not isinstance(model, Model):
        raise TypeError("Trainer requires a Model training root")
    return model


def _with_cp_topology(model: Model, metadata: Mapping[str, Any] | None):
    topology = model.context_parallel_context.checkpoint_topology()
    if topology is None:
        return metadata
    out = dict(metadata or {})
    mesh = dict(out.get("mesh") or {})
    mesh["context_parallel"] = topology
    out["mesh"] = mesh
    return out


class Trainer:
    def __init__(self, *, grad_accum_steps: int = 1, callbacks: CallbackGroup | None = None,
                 device: torch.device | str | None = None,
                 max_consecutive_skipped_updates: int | None = 64) -> None:
        if grad_accum_steps < 1:
            raise ValueError("grad_accum_steps must be at least one")
        self.grad_accum_steps = int(grad_accum_steps)
        # A run whose gradients stay non-finite would otherwise consume data forever without
        # advancing the iteration; None restores that behaviour.
        self.max_consecutive_skipped_updates = max_consecutive_skipped_updates
        self.periodic_iteration_offset = 0
        self.device = None if device is None else torch.device(device)
        if callbacks is None or not isinstance(callbacks, CallbackGroup):
            # a plain mapping/list from the config is turned into a group here
            config = None if callbacks is None else {"trainer": {"callbacks": callbacks}}
            callbacks = CallbackGroup(config=config, trainer=self)
        self.callbacks = callbacks
        self.callbacks.trainer = self
        for callback in self.callbacks:
            callback.trainer = self

    # ------------------------------------------------------------------------ data
    def _prepare(self, model: Model, batch: Batch) -> Batch:
        if self.device is not None:
            batch = to(batch, device=self.device)
        return model.prepare_data_batch(batch)

    def _next_batch(self, model: Model, iterator: Iterator[Batch], *, sequence_index: int):
        context = model.context_parallel_context
        batch, exhausted, owner = fetch_batch(context, iterator, sequence_index=sequence_index)
        if exhausted:
            return None
        return prepare_batch(context, batch, owner_rank=owner, prepare=partial(self._prepare, model))

    # ----------------------------------------------------------------------- train
    def train(self, model: Model, dataloader_train: Iterable[Batch],
              dataloader_val: Iterable[Batch] | None = None, *, grad_scaler: Any = None,
              max_iterations: int | None, checkpointer: Any = None,
              checkpoint_path: str | Path | None = None,
              checkpoint_components: Iterable[str] | None = None,
              checkpoint_optimizer_names: Iterable[str] | str | None = None,
              checkpoint_scheduler_names: Iterable[str] | str | None = None,
              checkpoint_model_key_prefix: str | None = None,
              checkpoint_interval: int | None = None, validation_interval: int | None = None,
              periodic_iteration_offset: int = 0, max_val_steps: int | None = None,
              validate_at_start: bool = False, save_final_checkpoint: bool = True,
              model_wrapper: Callable[[Model], torch.nn.Module] | None = None,
              runtime_metadata: Mapping[str, Any] | None = None,
              model_initializations: Any = None) -> int:
        """Run the loop; keyword names follow the ``train`` section of the config."""
        del model_initializations  # consumed by the entry point before training starts
        if periodic_iteration_offset < 0:
            raise ValueError("periodic_iteration_offset must be non-negative")
        self.periodic_iteration_offset = int(periodic_iteration_offset)
        scaler = grad_scaler if grad_scaler is not None else _NoScaler()
        try:
            iteration = self._loop(
                model, dataloader_train, dataloader_val, scaler, max_iterations, checkpointer,
                {"path": checkpoint_path, "components": checkpoint_components,
                 "optimizer_names": checkpoint_optimizer_names,
                 "scheduler_names": checkpoint_scheduler_names,
                 "model_key_prefix": checkpoint_model_key_prefix},
                checkpoint_interval, validation_interval, max_val_steps, validate_at_start,
                save_final_checkpoint, model_wrapper, _with_cp_topology(model, runtime_metadata))
        except BaseException as error:
            self._close(checkpointer, error)
            raise
        self._close(checkpointer, None)
        return iteration

    def _close(self, checkpointer, failure: BaseException | None) -> None:
        """Finish the pending checkpoint and release callbacks.  Nothing raised here may
        hide the training error; without one, the first cleanup error is raised."""
        problem: BaseException | None = None
        if checkpointer is not None:
            try:
                if failure is None:
                    checkpointer.finalize()
                else:
                    checkpointer.finalize_after_error()
            except BaseException as error:
                problem = error
                if failure is not None:
                    warnings.warn("Checkpoint finalization failed while handling a training "
                                  f"error: {type(error).__name__}: {error}", stacklevel=2)
        try:
            self.callbacks.on_app_end()
        except Exception as error:
            if failure is not None or problem is not None:
                warnings.warn(f"Callback cleanup failed: {type(error).__name__}: {error}",
                              stacklevel=2)
            else:
                problem = error
        if failure is None and problem is not None:
            raise problem

    def _restore(self, checkpointer, model, scaler, loader, options, metadata) -> int:
        kwargs = {"path": options["path"], "components": options["components"],
                  "dataloader": loader, "runtime_metadata": metadata}
        if options["model_key_prefix"] is not None:
            kwargs["model_key_prefix"] = options["model_key_prefix"]
        result = checkpointer.load(
            model,
            _pick(model.optimizer_dict, options["optimizer_names"], label="optimizer"),
            _pick(model.scheduler_dict, options["scheduler_names"], label="scheduler"),
            scaler, **kwargs)
        return result.iteration

    def _loop(self, model, loader, loader_val, scaler, max_iterations, checkpointer, load_options,
              checkpoint_interval, validation_interval, max_val_steps, validate_at_start,
              save_final, model_wrapper, metadata) -> int:
        iteration = 0
        if checkpointer is not None:
            iteration = self._restore(checkpointer, model, scaler, loader, load_options, metadata)

        def running() -> bool:
            return max_iterations is None or iteration < max_iterations

        def start_epoch() -> Iterator[Batch]:
            iterator = iter(loader)
            if checkpointer is not None:
                checkpointer.restore_pending_rng_state()  # after worker start-up
            return iterator

        def save() -> None:
            checkpointer.save(model, model.optimizer_dict, model.scheduler_dict, scaler,
                              iteration=iteration, dataloader=loader, runtime_metadata=metadata)

        def due(interval) -> bool:
            return model.is_cadence_due(iteration - self.periodic_iteration_offset, interval)

        wrapped = model if model_wrapper is None else model_wrapper(model)
        _root(wrapped)
        wrapped.train()
        self.callbacks.on_train_start(model, iteration=iteration)
        # Start the first epoch's workers before validation: sinks may start threads on
        # rank 0 and forking workers afterwards can deadlock that rank only.
        iterator = start_epoch() if running() else None
        if validate_at_start and loader_val is not None:
            self.validate(model, loader_val, iteration=iteration, max_val_steps=max_val_steps)

        accum, updates, last_saved, skipped = 0, 0, None, 0
        while running():
            if iterator is None:
                iterator = start_epoch()
            saw_batch = False
            while running():
                self.callbacks.on_before_dataloading(iteration=iteration)
                batch = self._next_batch(model, iterator,
                                         sequence_index=iteration * self.grad_accum_steps + accum)
                if batch is None:
                    break
                saw_batch = True
                if not wrapped.training:
                    wrapped.train()
                result = self.training_step(wrapped, scaler, batch, iteration=iteration,
                                            grad_accum_step=accum)
                accum = result.grad_accum_step
                if not result.did_update:
                    if result.found_nonfinite:
                        skipped += 1
                        limit = self.max_consecutive_skipped_updates
                        if limit is not None and skipped >= limit:
                            raise FloatingPointError(
                                f"{skipped} consecutive optimizer updates were skipped for non-finite "
                                f"gradients at iteration {iteration}")
                    continue
                skipped = 0
                iteration += 1
                updates += 1
                if checkpointer is not None and due(checkpoint_interval):
                    save()
                    last_saved = iteration
                if loader_val is not None and due(validation_interval):
                    if checkpointer is not None:
                        checkpointer.finalize()  # publish `latest` before a long evaluation
                    self.validate(model, loader_val, iteration=iteration,
                                  max_val_steps=max_val_steps)
            iterator = None
            if running() and not saw_batch:
                if is_rank0():
                    warnings.warn("Training dataloader produced no batches; ending training.",
                                  stacklevel=2)
                break
        if checkpointer is not None and save_final and updates > 0 and last_saved != iteration:
            save()
        self.callbacks.on_train_end(model, iteration=iteration)
        return iteration

    # ------------------------------------------------------------------------ step
    def training_step(self, model_ddp: torch.nn.Module, grad_scaler: Any, data_batch: Batch, *,
                      iteration: int = 0, grad_accum_step: int = 0) -> TrainingStepResult:
        """One microbatch: run the objective's loss closures (forward + backward each); on the
        last microbatch of an update also reduce, clip (callbacks), agree on finiteness, step
        and clear.  The hooks fire in the order the callback interface documents."""
        if grad_accum_step not in range(self.grad_accum_steps):
            raise ValueError(f"grad_accum_step must be in [0, {self.grad_accum_steps}), "
                             f"got {grad_accum_step}")
        scaler = _NoScaler() if grad_scaler is None else grad_scaler
        model = _root(model_ddp)
        bindings = model.get_optimizer_bindings(iteration)
        closes_update = grad_accum_step + 1 == self.grad_accum_steps
        self.callbacks.on_training_step_start(model, data_batch, iteration=iteration)
        outputs, loss = self._backward_passes(model_ddp, model, scaler, data_batch, iteration, closes_update)
        if not closes_update:
            self.callbacks.on_training_step_batch_end(model, data_batch, outputs, loss, iteration=iteration)
            return TrainingStepResult(outputs, loss, grad_accum_step + 1, did_update=False)
        nonfinite = self._update(model_ddp, bindings, scaler, loss.device, iteration)
        self.callbacks.on_training_step_batch_end(model, data_batch, outputs, loss, iteration=iteration)
        if not nonfinite:
            self.callbacks.on_training_step_end(model, data_batch, outputs, loss, iteration=iteration + 1)
        return TrainingStepResult(outputs, loss, 0, did_update=not nonfinite, found_nonfinite=nonfinite)

    def _backward_passes(self, model_ddp, model: Model, scaler, data_batch: Batch, iteration: int,
                         closes_update: bool) -> tuple[Batch, torch.Tensor]:
        """Every closure of the objective, forward and backward; returns the merged step
        outputs and the summed (detached) loss.  The objective must flag its last closure, and
        only that one: gradient synchronisation is switched on for exactly that backward."""
        outputs: Batch = {}
        losses: list[torch.Tensor] = []
        saw_last = False
        for _role, closure, is_last in model.training_step_closures(data_batch, iteration):
            if saw_last:
                raise RuntimeError("training_step_closures() produced another closure behind the one "
                                   "it flagged with is_last=True")
            if type(is_last) is not bool:
                raise TypeError("training_step_closures() must yield a bool as is_last, not "
                                f"{type(is_last).__name__}")
            saw_last = is_last
            final_backward = closes_update and is_last
            # from its last backward pass on, the sharded optimizer engines may reduce a layer's
            # gradients over the peers as soon as that layer's backward has finished
            zero.arm_overlap(final_backward)
            with ddp_sync_grad(model_ddp, final_backward):
                with span("forward"):
                    through_reducer = isinstance(model_ddp, DistributedDataParallel)
                    report, loss = model_ddp.forward_closure(closure) if through_reducer else closure()
                outputs.update(report)
                with span("backward"):
                    scaler.scale(loss / self.grad_accum_steps).backward()
            losses.append(loss.detach())
        if not losses:
            raise RuntimeError("training_step_closures() produced no closure at all")
        if not saw_last:
            raise RuntimeError("training_step_closures() never flagged a closure with is_last=True")
        total = losses[0]
        for more in losses[1:]:
            total = total + more
        return outputs, total

    def _update(self, model_ddp, bindings, scaler, device, iteration: int) -> bool:
        """Reduce, let callbacks clip, agree across ranks on finiteness, then step every active
        role or skip all of them; clear gradients either way.  Returns True when skipped."""
        hooks = self.callbacks
        optimizers = tuple(binding.optimizer for binding in bindings)
        for optimizer in optimizers:
            scaler.unscale_(optimizer)
            if callable(getattr(optimizer, "reduce_gradients", None)):
                optimizer.reduce_gradients()  # data-parallel mean (idempotent per update)
        for binding in bindings:
            hooks.on_before_optimizer_step(model_ddp, binding.optimizer, binding.scheduler, scaler,
                                           iteration=iteration)
        nonfinite = synchronize_found_nonfinite(scaler, optimizers, fallback_device=device)
        if nonfinite:
            hooks.on_optimizer_step_skipped(model_ddp, tuple(binding.name for binding in bindings),
                                            iteration=iteration)
        for binding in bindings if not nonfinite else ():
            with span(f"optimizer {binding.name}"):
                scaler.step(binding.optimizer)
            binding.scheduler.step()
            hooks.on_after_optimizer_step(model_ddp, binding.name, binding.optimizer, binding.scheduler,
                                          iteration=iteration)
        for binding in bindings:
            hooks.on_before_zero_grad(model_ddp, binding.optimizer, binding.scheduler, iteration=iteration)
            binding.optimizer.zero_grad(set_to_none=True)
            if hasattr(binding.optimizer, "grad_scale"):
                binding.optimizer.grad_scale = 1.0   # the clip coefficient applies to one update
        scaler.update()  # one scaler serves all roles: exactly once per update
        return nonfinite

    # -------------------------------------------------------------------- validate
    @torch.no_grad()
    def validate(self, model: Model, dataloader_val: Iterable[Batch], *, iteration: int = 0,
                 max_val_steps: int | None = None) -> None:
        with preserve_training_mode(model), _keep_loader_cursor(dataloader_val), isolated_rng():
            self.callbacks.on_validation_start(model, dataloader_val, iteration=iteration)
            model.eval()
            iterator = iter(dataloader_val)
            index = 0
            while max_val_steps is None or index < max_val_steps:
                batch = self._next_batch(model, iterator, sequence_index=index)
                if batch is None:
                    break
                outputs, loss = model.validation_step(batch, iteration)
                self.callbacks.on_validation_step_end(model, batch, outputs, loss,
                                                      iteration=iteration)
                index += 1
            self.callbacks.on_validation_end(model, iteration=iteration)
