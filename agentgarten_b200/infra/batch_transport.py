"""Delivery of training batches to ranks, with failures raised on every rank.

Without context parallelism each rank reads its own batch, but all ranks still agree on
OK / STOP / ERROR with an all-reduce(MAX), so an exception in one rank's dataset surfaces
everywhere instead of leaving the others blocked in the next collective.

With context parallelism the ranks of a CP group must see the *same* sample: microbatch
``i`` is read and prepared (device move + latent encoding) by group member ``i % cp`` and
shipped to the others.  The payload travels as one pickled skeleton (containers and
non-tensor leaves, tensors replaced by numbered slots) and ONE packed byte buffer holding
every tensor, followed by the owner's Python/NumPy/torch RNG state so that all members
continue with identical random streams.

Parity: reference ``wm/infra/batch_transport.py:63-317`` (which broadcasts tensor by tensor).
"""

from __future__ import annotations

import pickle
import random
from collections.abc import Callable, Iterator, Mapping
from dataclasses import dataclass
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

__all__ = ["fetch_batch", "prepare_batch"]

OK, STOP, ERROR = 0, 1, 2
Batch = dict[str, Any]


@dataclass(frozen=True)
class _Slot:
    index: int


def _on() -> bool:
    return dist.is_available() and dist.is_initialized()


def _wire_device() -> torch.device:
    if "nccl" in str(dist.get_backend()).lower():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _brief(error: BaseException) -> str:
    return f"{type(error).__name__}: {' '.join(str(error).split())[:400]}"


# ------------------------------------------------------------------ tree <-> buffer
def _strip(tree: Any, tensors: list[torch.Tensor], seen: dict[int, int]) -> Any:
    if torch.is_tensor(tree):
        if id(tree) not in seen:
            seen[id(tree)] = len(tensors)
            tensors.append(tree.detach())
        return _Slot(seen[id(tree)])
    if isinstance(tree, Mapping):
        items = [(k, _strip(v, tensors, seen)) for k, v in tree.items()]
        try:
            return type(tree)(items)
        except TypeError:
            return dict(items)
    if isinstance(tree, tuple) and hasattr(tree, "_fields"):
        return type(tree)(*(_strip(v, tensors, seen) for v in tree))
    if isinstance(tree, (list, tuple)):
        return type(tree)(_strip(v, tensors, seen) for v in tree)
    return tree


def _fill(tree: Any, tensors: list[torch.Tensor]) -> Any:
    if isinstance(tree, _Slot):
        return tensors[tree.index]
    if isinstance(tree, Mapping):
        items = [(k, _fill(v, tensors)) for k, v in tree.items()]
        try:
            return type(tree)(items)
        except TypeError:
            return dict(items)
    if isinstance(tree, tuple) and hasattr(tree, "_fields"):
        return type(tree)(*(_fill(v, tensors) for v in tree))
    if isinstance(tree, (list, tuple)):
        return type(tree)(_fill(v, tensors) for v in tree)
    return tree


def _layout(specs: list[tuple[tuple[int, ...], torch.dtype]]) -> tuple[list[int], int]:
    offsets, total = [], 0
    for shape, dtype in specs:
        offsets.append(total)
        nbytes = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
        total += -(-nbytes // 16) * 16
    return offsets, total


def _pack(tensors: list[torch.Tensor], device: torch.device):
    specs = [(tuple(int(s) for s in t.shape), t.dtype) for t in tensors]
    offsets, total = _layout(specs)
    buffer = torch.empty(max(total, 16), dtype=torch.uint8, device=device)
    for t, off in zip(tensors, offsets):
        flat = t.to(device).contiguous().view(-1).view(torch.uint8)
        buffer[off: off + flat.numel()].copy_(flat)
    return specs, buffer


def _unpack(specs, buffer: torch.Tensor) -> list[torch.Tensor]:
    offsets, _ = _layout(specs)
    out = []
    for (shape, dtype), off in zip(specs, offsets):
        nbytes = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
        out.append(buffer[off: off + nbytes].clone().view(dtype).view(shape))
    return out


# ----------------------------------------------------------------------- RNG handoff
def _rng_snapshot():
    cuda = None
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        cuda = torch.cuda.get_rng_state(torch.cuda.current_device()).cpu()
    return random.getstate(), np.random.get_state(), torch.get_rng_state(), cuda


def _rng_adopt(state) -> None:
    py, npy, cpu, cuda = state
    random.setstate(py)
    np.random.set_state(npy)
    torch.set_rng_state(cpu)
    if cuda is not None:
        torch.cuda.set_rng_state(cuda, torch.cuda.current_device())


# ---------------------------------------------------------------------- status sync
def _agree(status: int, rank: int | None, message: str | None):
    """World-wide MAX over status; on ERROR the lowest failing rank's message wins."""
    if not _on():
        return status, rank, message
    world = dist.get_world_size()
    word = torch.tensor([status, world - int(rank) if status == ERROR else 0],
                        dtype=torch.int64, device=_wire_device())
    dist.all_reduce(word, op=dist.ReduceOp.MAX)
    status, source = (int(v) for v in word.tolist())
    if status == ERROR:
        rank = world - source
        box = [message if dist.get_rank() == rank else None]
        dist.broadcast_object_list(box, src=rank)
        message = box[0]
    return status, rank, message


def _raise(status, rank, message, cause, stage: str) -> None:
    if status == ERROR:
        detail = "" if message is None else f": rank {int(rank)}: {message}"
        raise RuntimeError(f"Distributed dataloader {stage} failed{detail}") from cause


# --------------------------------------------------------------------------- public
def fetch_batch(context, iterator: Iterator[Batch], *, sequence_index: int):
    """Next batch → ``(batch on the reading rank, exhausted, owner rank in the CP group)``."""
    if not context.enabled and not _on():
        try:
            return next(iterator), False, None
        except StopIteration:
            return None, True, None
    owner = int(sequence_index) % context.size if context.enabled else None
    batch, status, rank, message, cause = None, OK, None, None, None
    if not context.enabled or context.rank == owner:
        try:
            batch = next(iterator)
        except StopIteration:
            status = STOP
        except BaseException as error:
            cause, status, rank, message = error, ERROR, dist.get_rank(), _brief(error)
    if context.enabled:
        box = [status, rank, message]
        context.broadcast_objects(box, source_rank=owner)
        status, rank, message = box
    status, rank, message = _agree(int(status), rank, message)
    _raise(status, rank, message, cause, "fetch")
    if status == STOP:
        return None, True, owner
    return batch, False, owner


def prepare_batch(context, data_batch: Batch | None, *, owner_rank: int | None,
                  prepare: Callable[[Batch], Batch]) -> Batch:
    """Run ``prepare`` where the batch was read; share the result inside the CP group."""
    if not context.enabled and not _on():
        return prepare(data_batch)
    status, rank, message, cause = OK, None, None, None
    prepared = skeleton = specs = rng = buffer = None
    device = _wire_device()
    mine = not context.enabled or context.rank == owner_rank
    if mine:
        try:
            prepared = prepare(data_batch)
            if context.enabled:
                tensors: list[torch.Tensor] = []
                skeleton = _strip(prepared, tensors, {})
                pickle.dumps(skeleton)  # fail here, not inside the object broadcast
                specs, buffer = _pack(tensors, device)
                rng = _rng_snapshot()
        except BaseException as error:
            cause, status, rank, message = error, ERROR, dist.get_rank(), _brief(error)
            skeleton = specs = rng = None  # whatever failed must not ride on the status message
    if context.enabled:
        box = [status, rank, message, rng, skeleton, specs]
        context.broadcast_objects(box, source_rank=int(owner_rank))
        status, rank, message, rng, skeleton, specs = box
    status, rank, message = _agree(int(status), rank, message)
    _raise(status, rank, message, cause, "prepare")
    if not context.enabled:
        return prepared
    if not mine:
        _, total = _layout(specs)
        buffer = torch.empty(max(total, 16), dtype=torch.uint8, device=device)
    from agentgarten_b200.parallel import switch_share

    if not switch_share.broadcast(buffer, int(owner_rank), context.group):  # multicast stores in a node
        dist.broadcast(buffer, src=context.global_rank(int(owner_rank)), group=context.group)
    _rng_adopt(rng)
    return _fill(skeleton, _unpack(specs, buffer))
