"""Periodic sampling during training.

On cadence (asked of the model, which may count something other than raw iterations; the
start-up validation at iteration 0 always samples) the callback runs ``model.sample`` on the
current training batch or on the first ``max_batches`` validation batches, under an
isolated RNG so that enabling previews never changes the training or validation streams.
With context parallelism only the group leader writes, under a rank index that numbers the
groups.  A failing writer is switched off; sampling never discards a model update.

Parity: reference ``wm/infra/callbacks/sampling.py:23-359``.
"""

from __future__ import annotations

import time
from collections.abc import Mapping, Sequence
from typing import Any, Protocol

import torch

from agentgarten_b200.infra.distributed import get_rank
from agentgarten_b200.infra.model import LifecycleCadence
from agentgarten_b200.infra.rng_state import isolated_rng
from agentgarten_b200.utils import log
from agentgarten_b200.utils.misc import map_tensors, preserve_training_mode

from .base import Callback

__all__ = ["ArtifactWriter", "ArtifactWriterGroup", "PeriodicSampleCallback"]


class ArtifactWriter(Protocol):
    def write(self, value: Any, *, output_dir: str, split: str, iteration: int, rank: int,
              sample_batch_index: int = 0) -> None: ...


def _close_quietly(writer: Any) -> None:
    close = getattr(writer, "close", None)
    if callable(close):
        try:
            close()
        except Exception as error:
            log.warning(f"Failed to close artifact writer {type(writer).__name__}: "
                        f"{type(error).__name__}: {error}")


class ArtifactWriterGroup:
    """Fans one artifact out to several writers; a writer that raises is disabled."""

    def __init__(self, writers: Sequence[ArtifactWriter | None]) -> None:
        self.writers = tuple(w for w in writers if w is not None)
        self._dead: set[int] = set()

    def write(self, value: Any, **where: Any) -> None:
        for writer in self.writers:
            if id(writer) in self._dead:
                continue
            try:
                writer.write(value, **where)
            except Exception as error:
                self._dead.add(id(writer))
                log.warning(f"Disabling artifact writer {type(writer).__name__} after write "
                            f"failure: {type(error).__name__}: {error}")

    def close(self) -> None:
        for writer in self.writers:
            _close_quietly(writer)


def _seed_of(value: Any) -> int | tuple[int, ...]:
    if torch.is_tensor(value):
        items = value.detach().cpu().reshape(-1).tolist()
    elif isinstance(value, (list, tuple)):
        items = list(value)
    else:
        return int(value)
    if not items:
        raise ValueError("sample seed batch metadata must not be empty")
    seeds = tuple(int(v) for v in items)
    return seeds[0] if len(seeds) == 1 else seeds


class PeriodicSampleCallback(Callback):
    def __init__(self, every_n: int | None, output_dir: str, writer: ArtifactWriter, *,
                 source: str = "validation", max_batches: int = 1,
                 sampling_options: Mapping[str, Any] | None = None,
                 seed_batch_key: str | None = "validation_sample_seed",
                 artifact_formatter: Any | None = None) -> None:
        super().__init__()
        if source not in ("train", "validation"):
            raise ValueError(f"sample source must be 'train' or 'validation', got {source!r}")
        if int(max_batches) < 0:
            raise ValueError(f"max_batches must be non-negative, got {max_batches}")
        self.every_n = None if every_n is None else int(every_n)
        self.output_dir, self.writer, self.source = str(output_dir), writer, source
        self.max_batches = int(max_batches)
        self.sampling_options = dict(sampling_options or {})
        self.seed_batch_key = None if seed_batch_key is None else str(seed_batch_key)
        self.artifact_formatter = artifact_formatter
        self._writer_ok = True
        self._pending = False
        self._index = 0

    def _due(self, iteration: int, model: Any = None) -> bool:
        if not self.every_n or self.every_n <= 0:
            return False
        if self.trainer is not None:
            iteration = int(iteration) - self.trainer.periodic_iteration_offset
        if int(iteration) == 0:
            return True
        if isinstance(model, LifecycleCadence):
            return bool(model.is_cadence_due(int(iteration), self.every_n))
        return int(iteration) % self.every_n == 0

    def _options(self, batch: Mapping[str, Any]) -> dict[str, Any]:
        options = dict(self.sampling_options)
        if self.seed_batch_key is not None and self.seed_batch_key in batch:
            options["seed"] = _seed_of(batch[self.seed_batch_key])
        return options

    def _emit(self, value: Any, model: Any, batch, split: str, iteration: int, index: int, options) -> None:
        if value is None or not self._writer_ok:
            return
        context = getattr(model, "context_parallel_context", None)
        if context is not None and not context.is_leader:
            return
        where = get_rank() if context is None else int(context.artifact_rank)
        try:
            if self.artifact_formatter is not None:
                value = self.artifact_formatter(value, model=model, data_batch=batch,
                                                sampling_options=options)
            self.writer.write(value, output_dir=self.output_dir, split=split, iteration=iteration,
                              rank=where, sample_batch_index=index)
        except Exception as error:
            self._writer_ok = False
            log.warning(f"Disabling artifact writer {type(self.writer).__name__} after write "
                        f"failure: {type(error).__name__}: {error}")

    def _sample(self, model: Any, data_batch, *, split: str, iteration: int, index: int = 0) -> None:
        begin = time.perf_counter()
        log.info(f"Sample start: split={split}, iteration={iteration}, batch={index}", rank0_only=False)
        try:
            with isolated_rng():
                batch = map_tensors(data_batch, lambda t: t.detach().clone())
                options = self._options(batch)
                with torch.inference_mode():
                    if split == "train":
                        with preserve_training_mode(model):
                            model.eval()
                            value = model.sample(batch, **options)
                    else:  # the trainer already put the model in eval mode
                        value = model.sample(batch, **options)
                self._emit(value, model, batch, split, iteration, index, options)
        except Exception:
            log.exception(f"Sample failed: split={split}, iteration={iteration}, batch={index}, "
                          f"elapsed_s={time.perf_counter() - begin:.3f}", rank0_only=False)
            raise
        log.info(f"Sample end: split={split}, iteration={iteration}, batch={index}, "
                 f"elapsed_s={time.perf_counter() - begin:.3f}", rank0_only=False)

    def on_training_step_end(self, model, data_batch, output_batch, loss, iteration=0):
        if self.source == "train" and self._due(iteration, model):
            self._sample(model, data_batch, split="train", iteration=iteration)

    def on_validation_start(self, model, dataloader_val, iteration=0):
        self._index = 0
        self._pending = self.source == "validation" and self.max_batches > 0 and self._due(iteration, model)

    def on_validation_step_end(self, model, data_batch, output_batch, loss, iteration=0):
        if not self._pending:
            return
        index = self._index
        self._index += 1
        if index >= self.max_batches:
            self._pending = False
            return
        # the batch was prepared (latents encoded) once for validation_step; reuse it
        self._sample(model, data_batch, split="validation", iteration=iteration, index=index)
        if self._index >= self.max_batches:
            self._pending = False

    def on_validation_end(self, model, iteration=0):
        self._pending, self._index = False, 0

    def on_app_end(self):
        _close_quietly(self.writer)
