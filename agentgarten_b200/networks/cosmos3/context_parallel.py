"""Ulysses context parallelism: tokens are sharded for all row-wise work, heads for attention.

Every chunk is split into ``ceil(N / cp)`` tokens per rank (zero padded).  Around attention
the ranks trade "all heads of my tokens" for "my heads of all tokens".  Unlike a per-chunk,
per-tensor exchange, q, k and v of **all chunks of the layer travel in one all-to-all** and
the attention outputs in a second one, so a 31-chunk teacher-forcing clip costs two
collectives per layer instead of 124.  KV heads are repeated when ``cp`` exceeds their
number; text keys/values are sliced by head locally.  The final hidden states are
all-gathered; since every rank of a group then evaluates the same loss, the backward of the
gather takes the local slice of the gradient times ``cp``.

Parity: reference ``wm/networks/cosmos3/context_parallel.py:20-140``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Any

import torch
import torch.distributed as dist

from .attention import TextContext

__all__ = ["ContextParallel", "ContextParallelAttention"]


def _all_to_all(value: torch.Tensor, group) -> torch.Tensor:
    """Within a node on CUDA: peer stores and counters (``parallel/peer_exchange.py``); else NCCL / Gloo."""
    from agentgarten_b200.parallel import peer_exchange

    value = value.contiguous()
    out = peer_exchange.exchange(value, group)
    if out is None:
        out = torch.empty_like(value)
        dist.all_to_all_single(out, value, group=group)
    return out


class _Exchange(torch.autograd.Function):
    """``out[s] = in_of_rank_s[my_rank]`` over dim 0; its own transpose, hence its backward."""

    @staticmethod
    def forward(ctx, value: torch.Tensor, group) -> torch.Tensor:
        ctx.group = group
        return _all_to_all(value, group)

    @staticmethod
    def backward(ctx, grad: torch.Tensor):
        return _all_to_all(grad, ctx.group), None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, value: torch.Tensor, group, rank: int, size: int) -> torch.Tensor:
        ctx.rank, ctx.size, ctx.local = rank, size, value.shape[1]
        from agentgarten_b200.parallel import switch_share

        stacked = switch_share.all_gather(value, group)   # one launch through the switch, or None
        if stacked is not None:
            return stacked.movedim(0, 1).reshape(value.shape[0], size * value.shape[1], *value.shape[2:])
        parts = [torch.empty_like(value) for _ in range(size)]
        dist.all_gather(parts, value.contiguous(), group=group)
        return torch.cat(parts, dim=1)

    @staticmethod
    def backward(ctx, grad: torch.Tensor):
        mine = grad.narrow(1, ctx.rank * ctx.local, ctx.local)
        return mine * ctx.size, None, None, None


def _pad_tokens(value: torch.Tensor, tokens: int) -> torch.Tensor:
    if value.shape[1] == tokens:
        return value
    return torch.nn.functional.pad(value, (0, 0) * (value.ndim - 2) + (0, tokens - value.shape[1]))


def _repeat(value: torch.Tensor, times: int) -> torch.Tensor:
    return value if times == 1 else value.repeat_interleave(times, dim=2)


@dataclass(frozen=True)
class ContextParallel:
    mesh: Any
    num_attention_heads: int
    num_key_value_heads: int

    def __post_init__(self) -> None:
        if self.num_attention_heads % self.size:
            raise ValueError(f"{self.num_attention_heads} query heads do not split over CP {self.size}")
        if (self.num_key_value_heads * self.kv_repeats) % self.size:
            raise ValueError(f"{self.num_key_value_heads} KV heads do not split over CP {self.size}")

    @property
    def group(self):
        return self.mesh.get_group()

    @property
    def size(self) -> int:
        return self.mesh.size()

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group)

    @property
    def kv_repeats(self) -> int:
        return max(self.size // self.num_key_value_heads, 1)

    def shard(self, value: torch.Tensor) -> torch.Tensor:
        local = math.ceil(value.shape[1] / self.size)
        return _pad_tokens(value, local * self.size).narrow(1, self.rank * local, local)

    def gather(self, value: torch.Tensor, tokens: int) -> torch.Tensor:
        return _Gather.apply(value, self.group, self.rank, self.size)[:, :tokens]

    # One exchange for a list of per-chunk tensors that share batch and head_dim.
    def heads_of_all_tokens(self, groups: list[list[torch.Tensor]], tokens: list[int],
                            ) -> list[list[torch.Tensor]]:
        """``groups[g][c]`` is ``[B, n_c, H_g, D]`` (local tokens, all heads) → same nesting
        with ``[B, N_c, H_g / cp, D]`` (all tokens, local heads)."""
        cp = self.size
        local = [g[0].shape[1] for g in zip(*groups)]
        heads = [g[0].shape[2] // cp for g in groups]
        stacked = []
        for g, h in zip(groups, heads):
            rows = torch.cat(g, dim=1)                                  # [B, n_tot, cp*h, D]
            b, n, _, d = rows.shape
            stacked.append(rows.view(b, n, cp, h, d))
        send = torch.cat(stacked, dim=3).permute(2, 0, 1, 3, 4)          # [cp, B, n_tot, sum_h, D]
        recv = _Exchange.apply(send, self.group)                         # dim 0 = source rank
        out: list[list[torch.Tensor]] = []
        for piece in recv.split(heads, dim=3):
            per_chunk = []
            for chunk, full in zip(piece.split(local, dim=2), tokens):
                # [cp, B, n_c, h, D] → [B, cp * n_c, h, D], source-rank major = token order
                joined = chunk.permute(1, 0, 2, 3, 4).flatten(1, 2)
                per_chunk.append(joined[:, :full])
            out.append(per_chunk)
        return out

    def tokens_of_all_heads(self, outputs: list[torch.Tensor], local: list[int]) -> list[torch.Tensor]:
        """Inverse for attention outputs: ``[B, N_c, H/cp, D]`` → ``[B, n_c, H, D]``."""
        cp = self.size
        padded = [_pad_tokens(o, n * cp) for o, n in zip(outputs, local)]
        # destination-rank major: rank r gets rows [r*n_c, (r+1)*n_c) of every chunk
        send = torch.cat([p.unflatten(1, (cp, n)) for p, n in zip(padded, local)], dim=2)
        send = send.permute(1, 0, 2, 3, 4)                               # [cp, B, n_tot, h, D]
        recv = _Exchange.apply(send, self.group)                         # dim 0 = source = head group
        merged = recv.permute(1, 2, 0, 3, 4).flatten(2, 3)               # [B, n_tot, cp*h, D]
        return list(merged.split(local, dim=1))

    # Per-tensor forms (kept for API parity and tests).
    def to_heads(self, value: torch.Tensor, tokens: int, *, kv: bool) -> torch.Tensor:
        if kv:
            value = _repeat(value, self.kv_repeats)
        return self.heads_of_all_tokens([[value]], [tokens])[0][0]

    def to_tokens(self, value: torch.Tensor, local_tokens: int) -> torch.Tensor:
        return self.tokens_of_all_heads([value], [local_tokens])[0]

    def text(self, text: TextContext) -> TextContext:
        heads = self.num_key_value_heads * self.kv_repeats // self.size
        lo = self.rank * heads
        return replace(
            text,
            keys=tuple(_repeat(k, self.kv_repeats)[:, :, lo:lo + heads] for k in text.keys),
            values=tuple(_repeat(v, self.kv_repeats)[:, :, lo:lo + heads] for v in text.values))


@dataclass
class ContextParallelAttention:
    """Wraps an attention policy: exchange in, inner policy on local heads, exchange out."""

    inner: Any
    cp: ContextParallel
    tokens: list[int]  # unsharded token count of every chunk

    def __call__(self, layer: int, queries, keys, values):
        cp = self.cp
        rep = cp.kv_repeats
        q, k, v = cp.heads_of_all_tokens(
            [list(queries), [_repeat(x, rep) for x in keys], [_repeat(x, rep) for x in values]],
            self.tokens)
        outputs = self.inner(layer, q, k, v)
        return cp.tokens_of_all_heads(outputs, [x.shape[1] for x in queries])
