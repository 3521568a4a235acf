"""Lifecycle hooks of the trainer.

A :class:`Callback` overrides any of 14 hooks; :class:`CallbackGroup` builds the callbacks
named in ``config.trainer.callbacks`` (an ordered mapping or a list; a ``null`` entry
disables a callback from the command line) and forwards every hook in configuration order.
``on_app_end`` reaches every callback even if an earlier one raises.

Parity: reference ``wm/infra/callbacks/base.py:29-209``.
"""

from __future__ import annotations

from collections.abc import Iterator, Mapping, Sequence
from typing import Any

from agentgarten_b200.infra.config import instantiate

__all__ = ["HOOKS", "Callback", "CallbackGroup"]

HOOKS = (
    "on_train_start", "on_before_dataloading", "on_training_step_start",
    "on_before_optimizer_step", "on_after_optimizer_step", "on_optimizer_step_skipped",
    "on_before_zero_grad", "on_training_step_batch_end", "on_training_step_end",
    "on_validation_start", "on_validation_step_end", "on_validation_end", "on_train_end",
    "on_app_end",
)


class Callback:
    """Base class: every hook is a no-op.

    ``on_training_step_batch_end`` fires once per microbatch; ``on_training_step_end`` once
    per successful optimizer update with ``iteration`` counting updates.
    """

    def __init__(self) -> None:
        self.config: Any | None = None
        self.trainer: Any | None = None

    def on_train_start(self, model, iteration=0): ...
    def on_before_dataloading(self, iteration=0): ...
    def on_training_step_start(self, model, data, iteration=0): ...
    def on_before_optimizer_step(self, model_ddp, optimizer, scheduler, grad_scaler, iteration=0): ...
    def on_after_optimizer_step(self, model_ddp, name, optimizer, scheduler, iteration=0): ...
    def on_optimizer_step_skipped(self, model_ddp, optimizer_names, iteration=0): ...
    def on_before_zero_grad(self, model_ddp, optimizer, scheduler, iteration=0): ...
    def on_training_step_batch_end(self, model, data_batch, output_batch, loss, iteration=0): ...
    def on_training_step_end(self, model, data_batch, output_batch, loss, iteration=0): ...
    def on_validation_start(self, model, dataloader_val, iteration=0): ...
    def on_validation_step_end(self, model, data_batch, output_batch, loss, iteration=0): ...
    def on_validation_end(self, model, iteration=0): ...
    def on_train_end(self, model, iteration=0): ...
    def on_app_end(self): ...


def _section(config: Any, name: str) -> Any:
    if config is None:
        return None
    return config.get(name) if isinstance(config, Mapping) else getattr(config, name, None)


class CallbackGroup(Callback):
    def __init__(self, config: Any | None, trainer: Any | None) -> None:
        super().__init__()
        self._callbacks: list[Callback] = []
        entries = _section(_section(config, "trainer"), "callbacks")
        if entries is None:
            return
        if isinstance(entries, Mapping):
            named = list(entries.items())
        elif isinstance(entries, Sequence) and not isinstance(entries, (str, bytes)):
            named = [(f"callback_{i}", entry) for i, entry in enumerate(entries)]
        else:
            raise TypeError("config.trainer.callbacks must be an ordered mapping or sequence, "
                            f"got {type(entries).__name__}")
        for name, entry in named:
            if entry is None:
                continue
            callback = entry if isinstance(entry, Callback) else instantiate(entry)
            if not isinstance(callback, Callback):
                raise TypeError(f"Callback {name!r} resolved to {type(callback).__name__}; "
                                "expected an instance of Callback")
            callback.config, callback.trainer = config, trainer
            self._callbacks.append(callback)

    @classmethod
    def of(cls, callbacks: Sequence[Callback], trainer: Any | None = None) -> "CallbackGroup":
        group = cls(None, trainer)
        for callback in callbacks:
            callback.trainer = trainer
            group._callbacks.append(callback)
        return group

    @property
    def callbacks(self) -> tuple[Callback, ...]:
        return tuple(self._callbacks)

    def __len__(self) -> int:
        return len(self._callbacks)

    def __iter__(self) -> Iterator[Callback]:
        return iter(self._callbacks)

    def on_app_end(self) -> None:
        errors: list[Exception] = []
        for callback in self._callbacks:
            try:
                callback.on_app_end()
            except Exception as error:  # keep going: cleanup must reach everyone
                errors.append(error)
        if len(errors) == 1:
            raise errors[0]
        if errors:
            raise ExceptionGroup("Callback cleanup failed", errors)


def _forward(name: str):
    def hook(group: CallbackGroup, *args: Any, **kwargs: Any) -> None:
        for callback in group:
            getattr(callback, name)(*args, **kwargs)

    hook.__name__ = name
    return hook


for _hook in HOOKS:
    if _hook != "on_app_end":
        setattr(CallbackGroup, _hook, _forward(_hook))
