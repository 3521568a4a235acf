"""Process-group bootstrap and data-parallel wrappers.

One process per GPU; rendezvous through ``env://`` (torchrun).  NCCL carries tensors on
CUDA, Gloo on CPU.  ``DistributedDataParallel`` here runs arbitrary loss closures inside
DDP's forward so that its reducer sees every backward.

Parity: reference ``wm/infra/distributed.py:34-249``.
"""

from __future__ import annotations

import os
from collections.abc import Callable, Iterator, Sequence
from contextlib import contextmanager
from datetime import timedelta
from typing import Any

import torch
import torch.distributed as dist

from agentgarten_b200.utils import log

__all__ = [
    "DistributedDataParallel",
    "ddp_sync_grad",
    "destroy_process_group",
    "get_local_rank",
    "get_local_world_size",
    "get_rank",
    "get_world_size",
    "init",
    "is_rank0",
    "wrap_ddp",
]


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def _resolve_device(device) -> torch.device:
    if device is None:
        return torch.device("cuda", get_local_rank()) if torch.cuda.is_available() \
            else torch.device("cpu")
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        return torch.device("cuda", get_local_rank())
    return device


def init(*, device=None, backend: str | None = None,
         timeout: timedelta = timedelta(minutes=30)) -> torch.device:
    """Bind this process to its device, then join the job's process group (if launched)."""
    device = _resolve_device(device)
    if dist.is_available() and dist.is_initialized():
        return device
    if device.type == "cuda":
        torch.cuda.set_device(device)  # before any PG or allocation
    if not dist.is_available() or "RANK" not in os.environ or "WORLD_SIZE" not in os.environ:
        return device
    backend = backend or ("nccl" if device.type == "cuda" else "gloo")
    if backend == "nccl" and device.type != "cuda":
        backend = "gloo"
    kwargs: dict[str, Any] = {}
    if device.type == "cuda":
        kwargs["device_id"] = device
    dist.init_process_group(backend=backend, init_method="env://", timeout=timeout, **kwargs)
    log.info(f"Initialized {backend} process group: rank={dist.get_rank()} "
             f"world_size={dist.get_world_size()} local_rank={get_local_rank()}",
             rank0_only=False)
    return device


def destroy_process_group() -> None:
    """Ends the process group.  The peer-memory links of this package are keyed by their group and
    hold symmetric buffers that were exchanged through it, so they are dropped first: a later
    ``init`` in the same process starts from fresh links."""
    if dist.is_available() and dist.is_initialized():
        import importlib

        for name in ("peer_exchange", "consensus", "switch_share"):
            try:
                importlib.import_module(f"agentgarten_b200.parallel.{name}").release()
            except Exception:  # a link that cannot be dropped must not keep the group alive
                pass
        dist.destroy_process_group()


def get_rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def get_world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def get_local_world_size() -> int:
    value = os.environ.get("LOCAL_WORLD_SIZE")
    return int(value) if value is not None else get_world_size()


def is_rank0() -> bool:
    return get_rank() == 0


class _ClosureRoot(torch.nn.Module):
    """DDP module whose forward executes a closure; parameters come from ``model``."""

    def __init__(self, model: torch.nn.Module) -> None:
        super().__init__()
        self.model = model

    def forward(self, closure: Callable[[], Any]) -> Any:
        return closure()


class DistributedDataParallel(torch.nn.parallel.DistributedDataParallel):
    def __init__(self, module: torch.nn.Module, *args: Any, **kwargs: Any) -> None:
        super().__init__(_ClosureRoot(module), *args, **kwargs)
        object.__setattr__(self, "training_model", module)
        self.show_sync_grad_static_graph_warning = True

    def forward_closure(self, closure: Callable[[], Any]) -> Any:
        return self(closure)


def wrap_ddp(model: torch.nn.Module, *, device=None, process_group=None,
             device_ids: Sequence[int] | None = None, output_device: int | None = None,
             find_unused_parameters: bool = False, static_graph: bool = False,
             broadcast_buffers: bool = True, gradient_as_bucket_view: bool = True):
    if not (dist.is_available() and dist.is_initialized()):
        return model
    if device is not None and device_ids is None:
        resolved = _resolve_device(device)
        if resolved.type == "cuda":
            device_ids = (resolved.index,)
            output_device = resolved.index if output_device is None else output_device
    return DistributedDataParallel(
        model, device_ids=device_ids, output_device=output_device, process_group=process_group,
        find_unused_parameters=find_unused_parameters, static_graph=static_graph,
        broadcast_buffers=broadcast_buffers, gradient_as_bucket_view=gradient_as_bucket_view)


@contextmanager
def ddp_sync_grad(model: torch.nn.Module, enabled: bool) -> Iterator[None]:
    """Enable/disable cross-replica gradient synchronisation for one backward.

    DDP: toggles the reducer.  Sharded engine: gradients are only reduced by the optimizer
    at the update boundary, so accumulation microbatches never communicate and nothing has
    to be toggled here.
    """
    if isinstance(model, DistributedDataParallel):
        before = model.require_backward_grad_sync
        if model.static_graph and before != enabled:
            if model.show_sync_grad_static_graph_warning and is_rank0():
                log.warning("DDP static_graph=True does not support changing gradient "
                            "synchronization; accumulation remains synchronized.")
            model.show_sync_grad_static_graph_warning = False
        else:
            model.require_backward_grad_sync = bool(enabled)
        try:
            yield
        finally:
            model.require_backward_grad_sync = before
        return
    yield
