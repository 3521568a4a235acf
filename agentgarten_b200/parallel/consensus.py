"""Small consensus values over the GPUs of a node through the NVSwitch (NVLS / ``multimem``).

``maximum(word)`` returns the element-wise maximum of a few non-negative numbers over all ranks:
the non-finite flag and the kernel status code that every update has to agree on.  Inside one
node whose GPUs share a multicast mapping it is one launch of ``csrc/multimem.cu`` (the switch
reduces and broadcasts); anywhere else (CPU, several nodes, no multicast support, or
``AGB200_MULTIMEM=0``) it is the library all-reduce, with the same result.

Parity: the one-element all-reduces of ``wm/infra/nonfinite.py:105-107``.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

__all__ = ["maximum", "release"]

_links: dict = {}
_LIMIT_NS = 30_000_000_000  # ranks reach an update at different times; the wait is bounded all the same


class _Link:
    def __init__(self, group, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.buffer = symm.empty(128, dtype=torch.int32, device=device)
        self.buffer.zero_()
        self.handle = symm.rendezvous(self.buffer, group=group)
        self.multicast = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.state = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # zeroed counters everywhere before the first arrival


def _link(group, device: torch.device):
    """The multicast link of this group, or None where the switch path does not apply."""
    if os.environ.get("AGB200_MULTIMEM", "1") == "0" or device.type != "cuda":
        return None
    key = (id(group), device.index)
    if key not in _links:
        link = None
        try:
            from agentgarten_b200.ops import native
            from agentgarten_b200.parallel.peer_exchange import _same_node

            world = dist.get_world_size(group)
            if native.available() and 1 < world <= 8 and dist.get_backend(group) == "nccl" and _same_node(group):
                link = _Link(group, device)
                if not link.multicast:
                    link = None
        except Exception:  # no symmetric memory, no multicast object: the library path serves
            link = None
        # every rank must take the same path
        verdict = torch.tensor([0 if link is None else 1], device=device)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=group)
        _links[key] = link if int(verdict.item()) == 1 else None
    return _links[key]


def maximum(word: torch.Tensor, group=None) -> torch.Tensor:
    """Element-wise maximum of ``word`` (up to 32 non-negative values below 2**24) over the ranks of
    ``group``; the result replaces ``word`` and is identical on every rank."""
    if not (dist.is_available() and dist.is_initialized()):
        return word
    group = dist.group.WORLD if group is None else group
    link = _link(group, word.device) if word.numel() <= 32 else None
    if link is None:
        dist.all_reduce(word, op=dist.ReduceOp.MAX, group=group)
        return word
    from agentgarten_b200.ops import native

    values = word.detach().to(torch.int32).contiguous()   # small non-negative integers: order-preserving
    out = torch.empty_like(values)
    native.count()
    native.ext().multimem_max(link.buffer, link.multicast, link.state, values, out, link.world, link.rank,
                              _LIMIT_NS)
    word.copy_(out.to(word.dtype))
    return word


def release() -> None:
    _links.clear()
