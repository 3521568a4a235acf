"""Gradient clipping with spike detection and per-role norms.

At an update boundary all active optimizer roles are measured and clipped once, as one
atomic update.  The global norm feeds an EMA-based spike detector (absolute threshold,
ratio to the EMA after a warm-up, or a non-finite norm).  A spike writes a JSON event per
rank with the metadata of the microbatches that produced it, and the step outputs gain
``metrics/grad_norm``, per-role norms, the clip coefficient and a spike flag.  A failing
event writer is switched off; monitoring never interrupts training.

Parity: reference ``wm/infra/callbacks/grad_monitor.py:43-308``.
"""

from __future__ import annotations

import json
import math
from collections.abc import Sequence
from typing import Any

import torch

from agentgarten_b200.infra.distributed import get_rank, is_rank0
from agentgarten_b200.utils import io, log

from .base import Callback
from .grad_clip import _check, clip_grad_norm_, clip_optimizers_

__all__ = ["GradClipMonitor"]


def _brief(value: Any) -> Any:
    if torch.is_tensor(value):
        return value.detach().cpu().tolist() if value.numel() <= 16 else f"tensor{tuple(value.shape)}"
    if isinstance(value, (str, int, float, bool)) or value is None:
        return value
    if isinstance(value, (list, tuple)) and len(value) <= 16:
        return [_brief(v) for v in value]
    return str(value)


class GradClipMonitor(Callback):
    def __init__(self, max_norm: float | None = 1.0, *, spike_threshold: float | None = None,
                 spike_ratio: float | None = 5.0, warmup_updates: int = 10, ema_decay: float = 0.95,
                 output_dir: str | None = None,
                 sample_keys: Sequence[str] = ("data_key", "latent_path", "sample_index",
                                               "caption_start_frame", "window_start_frame")) -> None:
        super().__init__()
        self.max_norm = None if max_norm is None else _check(max_norm)
        self.spike_threshold = None if spike_threshold is None else float(spike_threshold)
        self.spike_ratio = None if spike_ratio is None else float(spike_ratio)
        self.warmup_updates = max(0, int(warmup_updates))
        self.ema_decay = min(1.0, max(0.0, float(ema_decay)))
        self.output_dir = None if output_dir is None else str(output_dir)
        self.sample_keys = tuple(str(k) for k in sample_keys)
        self._samples: list[dict[str, Any]] = []
        self._ema: float | None = None
        self._seen = 0
        self._events = 0
        self._writer_ok = True
        self._reset()

    def _reset(self) -> None:
        self._measured = False
        self._norm: torch.Tensor | None = None
        self._role_norms: dict[str, torch.Tensor] = {}
        self._coefficient: float | None = None
        self._spike = False
        self._names: set[str] = set()

    def on_training_step_start(self, model, data, iteration=0):
        record = {k: _brief(data[k]) for k in self.sample_keys if k in data}
        if record:
            self._samples.append(record)

    def _judge(self, norm: float) -> tuple[bool, float | None]:
        before = self._ema
        finite = math.isfinite(norm)
        absolute = self.spike_threshold is not None and norm >= self.spike_threshold
        relative = (finite and self.spike_ratio is not None and self._seen >= self.warmup_updates
                    and before is not None and before > 0 and norm >= before * self.spike_ratio)
        if finite:
            self._ema = norm if before is None else self.ema_decay * before + (1 - self.ema_decay) * norm
        self._seen += 1
        return (not finite) or absolute or relative, before

    def _record_spike(self, iteration: int, norm: float, before: float | None) -> None:
        if self.output_dir is None or not self._writer_ok:
            return
        rank = get_rank()
        self._events += 1
        name = f"event_{self._events:06d}_iter_{iteration:09d}_rank_{rank:04d}.json"
        payload = {"iteration": iteration, "rank": rank, "grad_norm": norm,
                   "grad_norm_ema_before_update": before, "spike_threshold": self.spike_threshold,
                   "spike_ratio": self.spike_ratio, "microbatches": list(self._samples)}
        try:
            io.atomic_put_text(json.dumps(payload, ensure_ascii=False, sort_keys=True) + "\n",
                               io.join_path(self.output_dir, name))
        except Exception as error:
            self._writer_ok = False
            log.warning(f"Disabling gradient spike writer after failure: "
                        f"{type(error).__name__}: {error}")

    def _active(self, model_ddp, first_optimizer, iteration):
        root = getattr(model_ddp, "training_model", None) or model_ddp
        names_of = getattr(root, "get_optimizer_names", None)
        registry = getattr(root, "optimizer_dict", None)
        if not callable(names_of) or registry is None:
            return None
        names = tuple(names_of(iteration))
        if any(n not in registry for n in names) or all(registry[n] is not first_optimizer for n in names):
            return None
        return {str(n): registry[n] for n in names}

    def on_before_optimizer_step(self, model_ddp, optimizer, scheduler, grad_scaler, iteration=0):
        if self._measured:  # several active roles share one measurement
            return
        self._measured = True
        limit = float("inf") if self.max_norm is None else self.max_norm
        active = self._active(model_ddp, optimizer, iteration)
        if active is None:
            if getattr(optimizer, "engine", None) is not None:
                total, roles, _ = clip_optimizers_({"net": optimizer}, limit)
                roles = {}
            else:
                total, roles = clip_grad_norm_(model_ddp.parameters(), limit), {}
        else:
            total, roles, _ = clip_optimizers_(active, limit)
        if total is None:
            return
        self._norm = total.detach()
        self._role_norms = {r: n.detach() for r, n in roles.items()}
        norm = float(total.detach().float().cpu())  # the one host read of this callback
        if math.isinf(limit):
            self._coefficient = 1.0
        elif math.isfinite(norm):
            self._coefficient = min(1.0, self.max_norm / (norm + 1e-6))
        else:
            self._coefficient = 0.0
        self._spike, before = self._judge(norm)
        if self._spike:
            self._record_spike(iteration + 1, norm, before)
            if is_rank0():
                log.warning(f"Gradient spike at iteration {iteration + 1}: norm={norm:.6g}, "
                            f"previous_ema={before}")

    def on_after_optimizer_step(self, model_ddp, name, optimizer, scheduler, iteration=0):
        self._names.add(str(name))

    def on_optimizer_step_skipped(self, model_ddp, optimizer_names, iteration=0):
        self._names.update(optimizer_names)

    def on_training_step_batch_end(self, model, data_batch, output_batch, loss, iteration=0):
        if not self._measured:
            return
        if self._norm is not None:
            ref = self._norm
            output_batch["metrics/grad_norm"] = ref
            if self._role_norms:
                for role, norm in self._role_norms.items():
                    output_batch[f"metrics/{role}/grad_norm"] = norm
                    output_batch[f"metrics/{role}/grad_clip_coefficient"] = ref.new_tensor(self._coefficient)
            elif len(self._names) == 1:
                only = next(iter(self._names))
                if only != "net":
                    output_batch[f"metrics/{only}/grad_norm"] = ref
            output_batch["metrics/grad_clip_coefficient"] = ref.new_tensor(self._coefficient)
            output_batch["metrics/grad_spike"] = ref.new_tensor(float(self._spike))
        self._samples.clear()
        self._reset()
