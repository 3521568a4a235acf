"""Attention policies of the generation tower.

A policy is called once per layer with the per-chunk queries, keys and values
(``[B, N_c, H, D]`` each) and returns per-chunk outputs.  Every policy reduces to a *plan*:
for each query chunk, the ordered list of key/value chunks it may see (text keys come
first and are masked to each sample's prompt length).  The plan is executed by
:func:`agentgarten_b200.ops.planned_attention`, which on a B200 launches one segment-list
flash kernel over the concatenated chunks (no K/V concatenation per block, no mask
tensor) and elsewhere evaluates the same softmax chunk by chunk in PyTorch.

Because key tiles never straddle two chunks, a query row sees the same tile partition of
the same keys in ``forward_ar`` and in the cached rollout, which keeps the two bitwise
identical.

Parity: reference ``wm/networks/cosmos3/attention.py:27-300``.
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import TYPE_CHECKING, Any

import torch

from agentgarten_b200 import ops
from agentgarten_b200.protocols import HistoryWindow

if TYPE_CHECKING:
    from .network import Cosmos3Condition

__all__ = [
    "AnchorAttention",
    "BlockCausalAttention",
    "CachedAttention",
    "FullAttention",
    "HistoryWindow",
    "KVCache",
    "TextContext",
    "sdpa",
]

Chunks = list[torch.Tensor]


@dataclass(frozen=True)
class TextContext:
    """Per-layer keys/values of the prompt, ``[B, bucket, Hkv, D]``, plus real lengths."""

    keys: tuple[torch.Tensor, ...]
    values: tuple[torch.Tensor, ...]
    valid_lengths: torch.Tensor
    lengths: tuple[int, ...]

    @property
    def batch_size(self) -> int:
        return len(self.lengths)

    def repeat(self, times: int) -> "TextContext":
        if times == 1:
            return self
        return TextContext(
            keys=tuple(torch.cat((k,) * times) for k in self.keys),
            values=tuple(torch.cat((v,) * times) for v in self.values),
            valid_lengths=torch.cat((self.valid_lengths,) * times),
            lengths=self.lengths * times,
        )

    def head_slice(self, start: int, stop: int) -> "TextContext":
        return replace(
            self,
            keys=tuple(k[:, :, start:stop] for k in self.keys),
            values=tuple(v[:, :, start:stop] for v in self.values),
        )


def sdpa(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
         mask: torch.Tensor | None) -> torch.Tensor:
    """Attention on ``[B, N, H, D]`` tensors; ``mask`` is ``[B, 1, 1, NK]`` boolean or None.

    Forward-mode tangents on any input route through the attention-JVP operator.
    """
    key_mask = None if mask is None else mask.reshape(mask.shape[0], -1)
    return ops.attention(query, key, value, key_mask)


def _run(text: TextContext, layer: int, queries: Chunks, keys: Chunks, values: Chunks,
         plan: list[list[int]]) -> Chunks:
    return ops.planned_attention(
        queries, keys, values, plan,
        text_keys=text.keys[layer], text_values=text.values[layer],
        text_valid=text.valid_lengths)


@dataclass
class FullAttention:
    """Every query chunk sees the text and all visual chunks (bidirectional)."""

    text: TextContext

    def plan(self, chunks: int) -> list[list[int]]:
        return [list(range(chunks))] * chunks

    def __call__(self, layer: int, queries: Chunks, keys: Chunks, values: Chunks) -> Chunks:
        return _run(self.text, layer, queries, keys, values, self.plan(len(queries)))


def block_causal_plan(chunks: int, teacher_forcing: bool, history: HistoryWindow,
                      ) -> list[list[int]]:
    """Key-chunk lists for ``[C0, (query, [publication])...]`` chunk layouts.

    Chunk 0 (the anchor) sees itself.  Every chunk of block ``b`` sees the anchor, the
    visible history (the last chunk of earlier blocks, filtered by ``history``) and itself.
    """
    stride = 2 if teacher_forcing else 1
    if (chunks - 1) % stride:
        raise ValueError("teacher forcing needs a publication chunk per query chunk")
    plan: list[list[int]] = [[0]]
    published: list[int] = []
    for start in range(1, chunks, stride):
        prefix = [0, *history.visible(published)]
        for index in range(start, start + stride):
            plan.append([*prefix, index])
        published.append(start + stride - 1)
    return plan


@dataclass
class BlockCausalAttention:
    text: TextContext
    teacher_forcing: bool
    history: HistoryWindow = field(default_factory=HistoryWindow)

    def plan(self, chunks: int) -> list[list[int]]:
        return block_causal_plan(chunks, self.teacher_forcing, self.history)

    def __call__(self, layer: int, queries: Chunks, keys: Chunks, values: Chunks) -> Chunks:
        return _run(self.text, layer, queries, keys, values, self.plan(len(queries)))


@dataclass
class KVCache:
    """Immutable rollout cache: anchor K/V per layer plus the blocks inside the window.

    ``blocks[i][layer] = (K, V)``; ``block_frames[i]`` are the absolute frame indices of
    stored block ``i``.  Positions of new chunks derive from ``frames_committed``, never
    from what is stored.
    """

    text: TextContext
    anchor: tuple[tuple[torch.Tensor, torch.Tensor], ...]
    blocks: tuple[tuple[tuple[torch.Tensor, torch.Tensor], ...], ...] = ()
    block_frames: tuple[range, ...] = ()
    history: HistoryWindow = field(default_factory=HistoryWindow)
    frames_committed: int = 0
    condition: "Cosmos3Condition | None" = None
    grid: tuple[int, int] = (0, 0)

    def prefix(self, layer: int) -> list[tuple[torch.Tensor, torch.Tensor, list[int]]]:
        out = [(*self.anchor[layer], [0])]
        for block, frames in zip(self.blocks, self.block_frames, strict=True):
            out.append((*block[layer], list(frames)))
        return out

    def committed(self, block: tuple[tuple[torch.Tensor, torch.Tensor], ...], frames: int,
                  ) -> "KVCache":
        first = 1 + self.frames_committed
        stored: list[Any] = [*zip(self.blocks, self.block_frames, strict=True),
                             (block, range(first, first + frames))]
        kept = self.history.visible(stored)
        return replace(
            self,
            blocks=tuple(kv for kv, _ in kept),
            block_frames=tuple(span for _, span in kept),
            frames_committed=self.frames_committed + frames,
        )


@dataclass
class CachedAttention:
    """One new chunk against ``[text, anchor, cached blocks..., itself]``."""

    cache: KVCache
    record: bool = False
    recorded: list[tuple[torch.Tensor, torch.Tensor]] = field(default_factory=list)

    def __call__(self, layer: int, queries: Chunks, keys: Chunks, values: Chunks) -> Chunks:
        (query,), (key,), (value,) = queries, keys, values
        prefix = self.cache.prefix(layer)
        pool_k = [k for k, _, _ in prefix] + [key]
        pool_v = [v for _, v, _ in prefix] + [value]
        out = _run(self.cache.text, layer, [query], pool_k, pool_v, [list(range(len(pool_k)))])
        if self.record:
            self.recorded.append((key, value))
        return out


@dataclass
class AnchorAttention:
    """The anchor frame against ``[text, itself]``; records its K/V for the cache."""

    text: TextContext
    recorded: list[tuple[torch.Tensor, torch.Tensor]] = field(default_factory=list)

    def __call__(self, layer: int, queries: Chunks, keys: Chunks, values: Chunks) -> Chunks:
        (key,), (value,) = keys, values
        self.recorded.append((key, value))
        return _run(self.text, layer, queries, keys, values, [[0]])
