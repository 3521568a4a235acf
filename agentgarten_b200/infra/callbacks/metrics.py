"""Scalar metrics: accumulate on the device, reduce across ranks at flush time.

Every ``metrics/<name>`` entry of a step's outputs and the loss are folded into running
``(sum, count, invalid)`` triples on the device — no host synchronisation per step.  Every
``every_n`` updates (and at the end of training / validation) the names are agreed on with
one object all-gather, the triples are packed into one ``[n, 3]`` tensor and all-reduced,
and rank 0 writes the means to the sinks: ``train/loss``, ``train/<name>``,
``validation/*``, learning-rate gauges ``train/[role/]scheduler/lr_i`` and, optionally,
``performance/update_time_s`` / ``performance/updates_per_s``.  Non-finite observations are
counted and excluded.  A sink that raises is disabled; logging never stops training.

Parity: reference ``wm/infra/callbacks/metrics.py:23-428``.
"""

from __future__ import annotations

import time
from collections.abc import Mapping, Sequence
from typing import Any, Protocol

import torch
import torch.distributed as dist

from agentgarten_b200.infra.distributed import is_rank0
from agentgarten_b200.utils import log

from .base import Callback

__all__ = ["LoguruMetricSink", "MetricSink", "ScalarMetricCallback"]

PREFIX = "metrics/"


class MetricSink(Protocol):
    def write(self, metrics: Mapping[str, float], *, iteration: int) -> None: ...


class LoguruMetricSink:
    """Writes one log line per flush."""

    def write(self, metrics: Mapping[str, float], *, iteration: int) -> None:
        body = " | ".join(f"{k}={v:.6g}" for k, v in sorted(metrics.items()))
        log.info(f"iteration={iteration} | {body}")


def _scalar(value: Any, like: torch.Tensor) -> torch.Tensor | None:
    if torch.is_tensor(value):
        return value.detach().reshape(()).float() if value.numel() == 1 else None
    if isinstance(value, (int, float)) and not isinstance(value, bool):
        return torch.tensor(float(value), dtype=torch.float32, device=like.device)
    return None


class _Tally:
    """name → device tensor ``[sum, count, invalid]``."""

    def __init__(self) -> None:
        self.rows: dict[str, torch.Tensor] = {}
        self.ignored: set[str] = set()

    def add(self, name: str, value: torch.Tensor, weight: torch.Tensor | None = None) -> None:
        ok = torch.isfinite(value)
        clean = torch.where(ok, value, torch.zeros_like(value))
        if weight is None:
            row = torch.stack((clean, ok.float(), (~ok).float()))
        else:
            w = weight.to(device=value.device, dtype=torch.float32)
            w = torch.where(torch.isfinite(w) & (w >= 0), w, torch.zeros_like(w))
            row = torch.stack((clean * w, ok.float() * w, ((~ok) & (w > 0)).float()))
        have = self.rows.get(name)
        if have is None:
            self.rows[name] = row
        else:
            if have.device != row.device:
                have = self.rows[name] = have.to(row.device)
            have.add_(row)

    def observe(self, outputs: Mapping[str, Any], loss: torch.Tensor, split: str,
                weight: torch.Tensor | None = None) -> None:
        loss_name = f"{split}/loss"
        value = _scalar(loss, loss)
        if value is None:
            self.ignored.add(f"{loss_name} (non-scalar loss)")
        else:
            self.add(loss_name, value, weight)
        for key, raw in outputs.items():
            if not isinstance(key, str) or not key.startswith(PREFIX):
                continue
            short = key[len(PREFIX):]
            if not short:
                self.ignored.add("metrics/ (empty metric name)")
                continue
            name = f"{split}/{short}"
            if name == loss_name:
                self.ignored.add(f"{key} (reserved; the callback records the provided loss)")
                continue
            value = _scalar(raw, loss)
            if value is None:
                self.ignored.add(f"{key} (expected one scalar tensor or number)")
                continue
            self.add(name, value, weight)

    def clear(self) -> None:
        self.rows.clear()
        self.ignored.clear()


class ScalarMetricCallback(Callback):
    def __init__(self, every_n: int | None = 100, sinks: Sequence[MetricSink | None] | None = None, *,
                 report_update_speed: bool = False) -> None:
        super().__init__()
        self.every_n = None if every_n is None else int(every_n)
        self.sinks = tuple(s for s in sinks if s is not None) if sinks is not None \
            else (LoguruMetricSink(),)
        self.report_update_speed = bool(report_update_speed)
        self._train, self._val = _Tally(), _Tally()
        self._gauges: dict[str, torch.Tensor] = {}
        self._warned: set[str] = set()
        self._dead_sinks: set[int] = set()
        self._window_start: float | None = None
        self._window_updates = 0
        self._lr_before: dict[int, tuple[torch.Tensor, ...]] = {}

    # ------------------------------------------------------------------ speed gauge
    def on_before_dataloading(self, iteration=0):
        if self.report_update_speed and self._window_start is None:
            self._window_start = time.perf_counter()

    def _speed(self) -> dict[str, float]:
        if self._window_start is None or self._window_updates == 0:
            return {}
        per_update = (time.perf_counter() - self._window_start) / self._window_updates
        self._window_start, self._window_updates = None, 0
        return {"performance/update_time_s": per_update, "performance/updates_per_s": 1.0 / per_update}

    # -------------------------------------------------------------------- LR gauges
    def on_before_optimizer_step(self, model_ddp, optimizer, scheduler, grad_scaler, iteration=0):
        self._lr_before[id(optimizer)] = tuple(
            g["lr"].detach().reshape(()).float().clone() if torch.is_tensor(g["lr"])
            else torch.tensor(float(g["lr"])) for g in optimizer.param_groups)

    def on_after_optimizer_step(self, model_ddp, name, optimizer, scheduler, iteration=0):
        prefix = "" if name == "net" else f"{name}/"
        for i, lr in enumerate(self._lr_before.pop(id(optimizer), ())):
            self._gauges[f"train/{prefix}scheduler/lr_{i}"] = lr

    def on_optimizer_step_skipped(self, model_ddp, optimizer_names, iteration=0):
        self._lr_before.clear()

    # ------------------------------------------------------------------------ flush
    def _emit(self, metrics: Mapping[str, float], iteration: int) -> None:
        for sink in self.sinks:
            if id(sink) in self._dead_sinks:
                continue
            try:
                sink.write(metrics, iteration=iteration)
            except Exception as error:
                self._dead_sinks.add(id(sink))
                log.warning(f"Disabling metric sink {type(sink).__name__} after write failure: "
                            f"{type(error).__name__}: {error}")

    def _flush(self, tally: _Tally, iteration: int, gauges: dict[str, torch.Tensor] | None = None,
               extra: Mapping[str, float] | None = None) -> None:
        gauges = gauges if gauges is not None else {}
        names = sorted(set(tally.rows) | set(gauges))
        ignored = sorted(tally.ignored)
        distributed = dist.is_available() and dist.is_initialized()
        if distributed:
            everyone: list[Any] = [None] * dist.get_world_size()
            dist.all_gather_object(everyone, (names, ignored))
            names = sorted({n for item in everyone if item for n in item[0]})
            ignored = sorted({m for item in everyone if item for m in item[1]})
            device = torch.device("cuda", torch.cuda.current_device()) \
                if dist.get_backend() == "nccl" else torch.device("cpu")
        else:
            device = next(iter(tally.rows.values())).device if tally.rows else torch.device("cpu")
        packed = torch.zeros((len(names), 3), dtype=torch.float32, device=device)
        for i, name in enumerate(names):
            if name in tally.rows:
                packed[i].copy_(tally.rows[name].to(device))
            elif name in gauges:
                g = gauges[name].to(device=device, dtype=torch.float32)
                ok = torch.isfinite(g)
                packed[i, 0] = torch.where(ok, g, torch.zeros_like(g))
                packed[i, 1], packed[i, 2] = ok.float(), (~ok).float()
        if names and distributed:
            dist.all_reduce(packed, op=dist.ReduceOp.SUM)
        tally.clear()
        gauges.clear()
        if not is_rank0():
            return
        for message in sorted(set(ignored) - self._warned):
            self._warned.add(message)
            log.warning(f"Ignoring callback metric {message}")
        metrics: dict[str, float] = {}
        bad: dict[str, int] = {}
        for name, (total, count, invalid) in zip(names, packed.cpu().tolist()):
            if count > 0:
                metrics[name] = total / count
            if invalid > 0:
                bad[name] = int(invalid)
        metrics.update(extra or {})
        if bad:
            log.warning(f"Excluded non-finite metric observations at iteration {iteration}: "
                        + ", ".join(f"{k}={v}" for k, v in sorted(bad.items())))
        if metrics:
            self._emit(metrics, iteration)

    # ------------------------------------------------------------------------ hooks
    def on_training_step_batch_end(self, model, data_batch, output_batch, loss, iteration=0):
        self._train.observe(output_batch, loss, "train")

    def on_training_step_end(self, model, data_batch, output_batch, loss, iteration=0):
        if self.report_update_speed:
            self._window_updates += 1
        if self.every_n and self.every_n > 0 and iteration % self.every_n == 0:
            self._flush(self._train, iteration, self._gauges, self._speed())

    def on_train_end(self, model, iteration=0):
        self._flush(self._train, iteration, self._gauges, self._speed())

    def on_validation_start(self, model, dataloader_val, iteration=0):
        self._val.clear()

    def on_validation_step_end(self, model, data_batch, output_batch, loss, iteration=0):
        weight = _scalar(data_batch.get("validation_metric_weight", 1.0), loss)
        if weight is None:
            self._val.ignored.add("validation_metric_weight (expected one scalar tensor or number)")
            weight = torch.zeros((), device=loss.device)
        self._val.observe(output_batch, loss, "validation", weight)

    def on_validation_end(self, model, iteration=0):
        self._flush(self._val, iteration)

    def on_app_end(self):
        for sink in self.sinks:
            close = getattr(sink, "close", None)
            if callable(close):
                try:
                    close()
                except Exception as error:
                    log.warning(f"Failed to close metric sink {type(sink).__name__}: "
                                f"{type(error).__name__}: {error}")
