"""Training entry point: ``python -m agentgarten_b200.train experiment=cosmos3/bidirectional ...``
(also reachable as ``python -m wm.train``).

Order: load ``.env`` (never overriding exported variables) → compose the configuration →
join the process group → publish the resolved ``config.yaml`` (rank 0 writes, every rank
learns whether it worked) → torch backend flags → seed (offset by rank) → build and place the
model → callbacks, trainer, checkpointer → initial weights → optimizers and schedulers →
re-seed → data loaders → ``Trainer.train``.  The process group is destroyed only if this
call created it.

Parity: reference ``wm/train.py:32-185``.
"""

from __future__ import annotations

import os
import sys
from collections.abc import Callable, Mapping, Sequence
from datetime import timedelta
from typing import Any

import torch
import torch.distributed as dist

from agentgarten_b200.configs.compose import EXPERIMENT_MODULE_ROOT, compose_config
from agentgarten_b200.infra import distributed
from agentgarten_b200.infra.callbacks import CallbackGroup
from agentgarten_b200.infra.config import instantiate, to_yaml
from agentgarten_b200.utils import io, log
from agentgarten_b200.utils.misc import set_random_seed

__all__ = ["main"]


def _load_dotenv(path: str = ".env") -> None:
    """KEY=VALUE lines; exported variables win."""
    if not os.path.isfile(path):
        return
    with open(path) as handle:
        for line in handle:
            line = line.strip()
            if not line or line.startswith("#") or "=" not in line:
                continue
            key, _, value = line.partition("=")
            key = key.removeprefix("export ").strip()
            value = value.strip().strip("'\"")
            os.environ.setdefault(key, value)


def _publish_resolved_config(config) -> None:
    problem: BaseException | None = None
    if distributed.is_rank0():
        try:
            io.atomic_put_text(to_yaml(config), io.join_path(config.job.output_dir, "config.yaml"))
        except BaseException as error:
            problem = error
    message = None if problem is None else f"{type(problem).__name__}: {' '.join(str(problem).split())[:400]}"
    if dist.is_available() and dist.is_initialized():
        box = [message]
        dist.broadcast_object_list(box, src=0)
        message = box[0]
    if message is not None:
        raise RuntimeError(f"Resolved config publication failed on rank 0: {message}") from problem


def _configure_torch(settings: Mapping[str, Any] | None) -> None:
    if not settings:
        return
    if "deterministic" in settings:
        torch.backends.cudnn.deterministic = bool(settings["deterministic"])
    if "benchmark" in settings:
        torch.backends.cudnn.benchmark = bool(settings["benchmark"])
    if "allow_tf32" in settings:
        torch.backends.cuda.matmul.allow_tf32 = bool(settings["allow_tf32"])
        torch.backends.cudnn.allow_tf32 = bool(settings["allow_tf32"])
    if "float32_matmul_precision" in settings:
        torch.set_float32_matmul_precision(settings["float32_matmul_precision"])
    # the ``compile`` sub-section is accepted for recipe compatibility; nothing is traced


def _seed(runtime: Mapping[str, Any]) -> None:
    if runtime.get("seed") is not None:
        set_random_seed(int(runtime["seed"]), by_rank=bool(runtime.get("seed_by_rank", False)))


def _model_wrapper(config: Mapping[str, Any] | None, device) -> Callable | None:
    if config is None:
        return None
    return lambda model: instantiate(config, model=model, device=device)


def _run(config, device: torch.device) -> int:
    model = instantiate(config.model)
    model.parallelize(device)
    callbacks = CallbackGroup(config, trainer=None)
    trainer = instantiate(config.trainer, callbacks=callbacks, device=device)
    checkpointer = instantiate(config.checkpoint)
    train_kwargs = dict(config.get("train", {}))
    components = train_kwargs.get("checkpoint_components")
    resuming = train_kwargs.get("checkpoint_path") is not None and (
        components is None or "model" in components)
    checkpointer.initialize_model(model, train_kwargs.pop("model_initializations", {}), resume=resuming)
    model.init_optimizer_scheduler(config.optimizer, config.scheduler)
    grad_scaler = instantiate(config.grad_scaler) if config.get("grad_scaler") is not None else None
    if grad_scaler is not None and device.type != "cuda" and not grad_scaler.is_enabled():
        grad_scaler = None
    _seed(config.get("runtime", {}))  # initialisation may have moved the per-rank streams
    loader_train = instantiate(config.dataloader_train)
    loader_val = None if config.get("dataloader_val") is None else instantiate(config.dataloader_val)
    return trainer.train(model, loader_train, loader_val, grad_scaler=grad_scaler,
                         checkpointer=checkpointer,
                         model_wrapper=_model_wrapper(config.get("model_wrapper"), device),
                         **train_kwargs)


def main(argv: Sequence[str] | None = None, *,
         experiment_module_root: str = EXPERIMENT_MODULE_ROOT) -> int:
    _load_dotenv()
    log.configure()
    config = compose_config(list(sys.argv[1:] if argv is None else argv),
                            experiment_module_root=experiment_module_root)
    runtime = config.get("runtime", {})
    owned = not (dist.is_available() and dist.is_initialized())
    device = distributed.init(
        device=runtime.get("device"), backend=runtime.get("backend"),
        timeout=timedelta(seconds=float(runtime.get("process_group_timeout_seconds", 300.0))))
    try:
        _publish_resolved_config(config)
        _configure_torch(runtime.get("torch"))
        _seed(runtime)
        return _run(config, device)
    finally:
        log.complete()
        if owned:
            distributed.destroy_process_group()


if __name__ == "__main__":
    main()
    raise SystemExit(0)
