"""All-to-all between the GPUs of one node over NVLink peer memory.

The Ulysses exchange of context parallelism (``wm/networks/cosmos3/context_parallel.py:20-60``
in the reference, an NCCL ``all_to_all_single``) as two kernels of this package
(``csrc/exchange.cu``): every rank stores its blocks straight into the receive buffers of
their destinations through the peer mapping and signals them with system-scope counters;
the receiver waits (bounded) for all blocks and copies them out.  The buffers are symmetric
memory, allocated once per process group and grown when a larger exchange comes along (all
ranks see the same sizes, so they grow together).

``exchange(value, group)`` returns ``None`` when the path does not apply (CPU tensors, one
rank, a group that spans nodes, no extension, or ``AGB200_NCCL_EXCHANGE=1``); the caller
then uses the library collective.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from agentgarten_b200.ops import native

__all__ = ["exchange", "release"]

_MIN_HALF_BYTES = 64 << 20
_links: dict = {}


class _Link:
    """Symmetric receive buffer, arrival counter and local state of one process group."""

    def __init__(self, group, device: torch.device, half_bytes: int) -> None:
        import torch.distributed._symmetric_memory as symm

        self.group, self.device, self.half_bytes = group, device, half_bytes
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.buffer = symm.empty(2 * half_bytes, dtype=torch.uint8, device=device)
        from .debug import poison

        poison(self.buffer)   # under AGB200_POISON=1: a block nobody stored reads as NaN
        self.counter = symm.empty(4, dtype=torch.int32, device=device)
        self.counter.zero_()
        self._handles = [symm.rendezvous(self.buffer, group=group), symm.rendezvous(self.counter, group=group)]
        self.recv_ptrs = [int(p) for p in self._handles[0].buffer_ptrs]
        self.arrive_ptrs = [int(p) for p in self._handles[1].buffer_ptrs]
        self.state = torch.zeros(2, dtype=torch.int32, device=device)  # exchanges done, ticket
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # zeroed counters everywhere before the first signal


def _same_node(group) -> bool:
    from agentgarten_b200.infra.distributed import get_local_world_size

    local = get_local_world_size()
    ranks = dist.get_process_group_ranks(group)
    return len({r // max(local, 1) for r in ranks}) == 1


def _link(group, device: torch.device, nbytes: int):
    key = (tuple(dist.get_process_group_ranks(group)), device.index)
    link = _links.get(key)
    if link is False:
        return None
    if link is None or link.half_bytes < nbytes:
        if link is None and not _same_node(group):
            _links[key] = False
            return None
        half = max(_MIN_HALF_BYTES, 1 << (nbytes - 1).bit_length())
        if link is not None:
            # every rank reaches this point for the same exchange: finish the old buffer first
            torch.cuda.synchronize(device)
            dist.barrier(group=group)
        try:
            link = _links[key] = _Link(group, device, half)
        except (RuntimeError, ImportError) as error:  # no symmetric memory for this group
            from agentgarten_b200.utils import log

            log.warning(f"peer-memory exchange unavailable ({error}); using the library collective")
            _links[key] = False
            return None
    return link


def exchange(value: torch.Tensor, group) -> torch.Tensor | None:
    """``out[s] = value_of_rank_s[my_rank]`` over dim 0 (``value`` is ``[world, ...]``), or ``None``."""
    if not value.is_cuda or os.environ.get("AGB200_NCCL_EXCHANGE") == "1":
        return None
    if os.environ.get("AGB200_DISABLE_NATIVE") == "1" or not dist.is_initialized():
        return None
    group = group if group is not None else dist.group.WORLD
    world = dist.get_world_size(group)
    if world < 2 or world > 8 or value.shape[0] != world or dist.get_backend(group) != "nccl":
        return None
    value = value.contiguous()
    nbytes = value.numel() * value.element_size()
    if nbytes == 0 or (nbytes // world) % 16:
        return None
    link = _link(group, value.device, nbytes)
    if link is None:
        return None
    out = torch.empty_like(value)
    native.count(2)
    native.ext().exchange(value, out, link.recv_ptrs, link.arrive_ptrs, link.state, link.half_bytes, link.rank)
    return out


def release() -> None:
    """Drop the symmetric buffers (before the process group goes away)."""
    _links.clear()
