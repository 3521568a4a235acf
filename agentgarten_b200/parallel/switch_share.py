"""All-gather and broadcast inside a node through NVSwitch multicast stores (NVLS / ``multimem``).

``all_gather(value)`` returns ``[world, *value.shape]`` and ``broadcast(buffer, source)`` fills
``buffer`` on every rank, each in one launch of ``csrc/multimem.cu``: a rank stores its bytes once
through the multicast mapping of a symmetric buffer (the switch delivers them to every GPU), all
CTAs of all ranks announce their stores on a counter in the same buffer, and each rank copies the
complete payload out of its own copy.  Both return ``None`` / ``False`` where the switch path does
not apply (CPU, several nodes, no multicast object, ``AGB200_MULTIMEM=0``); the caller then uses
the library collective, with the same result.

Used by the final-hidden gather of context parallelism and by the batch hand-over inside a
context-parallel group.

Parity: the ``all_gather`` of ``wm/networks/cosmos3/context_parallel.py:83-86`` and the tensor
broadcasts of ``wm/infra/batch_transport.py:312-314``.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

__all__ = ["all_gather", "broadcast", "release"]

_links: dict = {}
_LIMIT_NS = 30_000_000_000
_MIN_HALF = 32 << 20       # bytes per half of the first buffer of a group
_HEADER = 256              # counter block in front of the halves (csrc/multimem.cu)


class _Link:
    def __init__(self, group, device: torch.device, half_bytes: int) -> None:
        import torch.distributed._symmetric_memory as symm

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.buffer = symm.empty((_HEADER + 2 * half_bytes) // 4, dtype=torch.int32, device=device)
        self.buffer[: _HEADER // 4].zero_()
        self.handle = symm.rendezvous(self.buffer, group=group)
        self.multicast = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.state = torch.zeros(2, dtype=torch.int32, device=device)
        self.capacity = half_bytes
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # zeroed counters everywhere before the first arrival


def _round_up(value: int, to: int) -> int:
    return -(-value // to) * to


def _link(group, device: torch.device, total: int):
    """The link of this group with room for ``total`` bytes, or None where the switch path does
    not apply.  Creation (and growth) is collective: every rank calls with the same ``total``."""
    if os.environ.get("AGB200_MULTIMEM", "1") == "0" or device.type != "cuda":
        return None
    key = (id(group), device.index)
    known = _links.get(key, False)
    if known is None or (known and known.capacity >= total):
        return known
    link = None
    try:
        from agentgarten_b200.ops import native
        from agentgarten_b200.parallel.peer_exchange import _same_node

        world = dist.get_world_size(group)
        if native.available() and 1 < world <= 8 and dist.get_backend(group) == "nccl" and _same_node(group):
            half = max(_MIN_HALF, 1 << (total - 1).bit_length())
            if known:
                torch.cuda.synchronize(device)  # nothing of the smaller buffer is still in flight
            link = _Link(group, device, half)
            if not link.multicast:
                link = None
    except Exception:  # no symmetric memory, no multicast object: the library path serves
        link = None
    verdict = torch.tensor([0 if link is None else 1], device=device)
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=group)  # every rank takes the same path
    _links[key] = link if int(verdict.item()) == 1 else None
    return _links[key]


def _bytes_of(value: torch.Tensor) -> torch.Tensor:
    """``value`` as a flat byte tensor whose length and address are multiples of 16."""
    flat = value.contiguous().reshape(-1).view(torch.uint8)
    padded = _round_up(flat.numel(), 16)
    if padded != flat.numel() or flat.data_ptr() % 16:
        room = torch.empty(padded, dtype=torch.uint8, device=value.device)
        room[: flat.numel()].copy_(flat)
        return room
    return flat


def all_gather(value: torch.Tensor, group=None) -> torch.Tensor | None:
    """``[world, *value.shape]`` with slice ``r`` holding rank ``r``'s ``value`` (all ranks pass the
    same shape and dtype), or None where the switch path does not apply."""
    if not (dist.is_available() and dist.is_initialized()) or not value.is_cuda or value.numel() == 0:
        return None
    group = dist.group.WORLD if group is None else group
    world = dist.get_world_size(group)
    if world < 2:
        return None
    part = _bytes_of(value)
    link = _link(group, value.device, world * part.numel())
    if link is None:
        return None
    from agentgarten_b200.ops import native

    out = torch.empty(world * part.numel(), dtype=torch.uint8, device=value.device)
    native.count()
    native.ext().multimem_share(link.buffer, link.multicast, link.state, part, link.rank * part.numel(), out,
                                link.world, _LIMIT_NS)
    rows = out.view(world, part.numel())[:, : value.numel() * value.element_size()]
    if rows.shape[1] != part.numel():
        rows = rows.contiguous()
    return rows.view(value.dtype).view(world, *value.shape)


def broadcast(buffer: torch.Tensor, source: int, group=None) -> bool:
    """Fill the contiguous ``buffer`` of every rank with the one of group rank ``source``; False
    (nothing done) where the switch path does not apply."""
    if not (dist.is_available() and dist.is_initialized()) or not buffer.is_cuda or buffer.numel() == 0:
        return False
    if not buffer.is_contiguous():
        return False
    group = dist.group.WORLD if group is None else group
    if dist.get_world_size(group) < 2:
        return False
    flat = buffer.reshape(-1).view(torch.uint8)
    total = _round_up(flat.numel(), 16)
    link = _link(group, buffer.device, total)
    if link is None:
        return False
    from agentgarten_b200.ops import native

    mine = link.rank == int(source)
    part = _bytes_of(buffer) if mine else torch.empty(0, dtype=torch.uint8, device=buffer.device)
    whole = flat if total == flat.numel() and flat.data_ptr() % 16 == 0 else \
        torch.empty(total, dtype=torch.uint8, device=buffer.device)
    native.count()
    native.ext().multimem_share(link.buffer, link.multicast, link.state, part, 0, whole, link.world, _LIMIT_NS)
    if whole is not flat:
        flat.copy_(whole[: flat.numel()])
    return True


def release() -> None:
    _links.clear()
