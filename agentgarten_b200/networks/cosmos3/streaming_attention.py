"""Persistent per-layer K/V storage of one streaming sample.

Keys and values live in fixed arenas ``[1, text + (capacity + block) * frame_tokens, Hkv, D]``
that never move while a stream runs (stable addresses are what lets a whole denoise step
replay as a CUDA graph).  The current chunk's K/V are written behind the committed history;
attention reads ``[text | history | current]`` in place — on a B200 through the segment-list
flash kernel (text masked to the prompt length, no mask tensor, no concatenation).  FIFO
eviction with RoPE re-rotation goes to a second arena in one pass and the arenas swap.

Parity: reference ``wm/networks/cosmos3/streaming_attention.py:14-111``.
"""

from __future__ import annotations

import torch

from agentgarten_b200 import ops
from agentgarten_b200.ops import native

__all__ = ["StreamAttentionCache"]


class StreamAttentionCache:
    def __init__(self, text_k: torch.Tensor, text_v: torch.Tensor, frame_tokens: int, capacity: int,
                 block_frames: int) -> None:
        self.text_tokens = text_k.shape[1]
        self.frame_tokens = frame_tokens
        self.capacity = capacity
        self.block_frames = block_frames
        rows = self.text_tokens + (capacity + block_frames) * frame_tokens
        shape = (1, rows, *text_k.shape[2:])
        # zero-filled: tiles that overhang a segment multiply stale rows by probability 0
        self.key = text_k.new_zeros(shape)
        self.value = text_v.new_zeros(shape)
        self.key[:, : self.text_tokens].copy_(text_k)
        self.value[:, : self.text_tokens].copy_(text_v)
        self.frames = 0
        self._spare: tuple[torch.Tensor, torch.Tensor] | None = None
        self._swapped = False  # True while the second arena is the live one

    # ------------------------------------------------------------------------ views
    def _row_of_frame(self, frame: int) -> int:
        """Arena row at which visual frame ``frame`` starts (the text rows come first)."""
        return self.text_tokens + frame * self.frame_tokens

    @property
    def visual_key(self) -> torch.Tensor:
        return self.key[:, self.text_tokens: self._row_of_frame(self.frames)]

    @property
    def visual_value(self) -> torch.Tensor:
        return self.value[:, self.text_tokens: self._row_of_frame(self.frames)]

    def _write(self, first_row: int, key: torch.Tensor, value: torch.Tensor) -> int:
        """Copy a chunk's K/V into both arenas from ``first_row`` on; returns the row behind it."""
        behind = first_row + key.shape[1]
        self.key[:, first_row:behind].copy_(key)
        self.value[:, first_row:behind].copy_(value)
        return behind

    # ------------------------------------------------------------------------- use
    def attend(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        """Attention of an uncommitted chunk over text, committed history and itself.  The chunk
        is parked behind the history; ``frames`` is untouched, so nothing is committed."""
        behind = self._write(self._row_of_frame(self.frames), key, value)
        return ops.attention(query, self.key[:, :behind], self.value[:, :behind], None)

    def append(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """Commit a chunk: its K/V become history."""
        self._write(self._row_of_frame(self.frames), key, value)
        self.frames += key.shape[1] // self.frame_tokens

    def replace_visual(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """The whole history is replaced (eviction without re-rotation, or a rebuilt cache)."""
        self.frames = 0
        self.append(key, value)

    def relocate(self, sink_frames: int, evicted_frames: int,
                 rotation: tuple[torch.Tensor, torch.Tensor]) -> None:
        """Drop ``evicted_frames`` frames behind the sink and rotate the kept keys by
        ``rotation = (cos, sin)`` (FP32 ``[1, kept_tokens, D]``); values only move."""
        from agentgarten_b200.ops.kernels.stream_cache import relocate

        if self._spare is None:
            self._spare = torch.zeros_like(self.key), torch.zeros_like(self.value)
        text, sink = self.text_tokens, sink_frames * self.frame_tokens
        shift = evicted_frames * self.frame_tokens
        used = text + self.frames * self.frame_tokens
        key, value = self._spare
        key[:, :text].copy_(self.key[:, :text])
        value[:, :text].copy_(self.value[:, :text])
        relocate(self.key[:, text:used], key[:, text:], sink, shift, rotation)
        relocate(self.value[:, text:used], value[:, text:], sink, shift)
        self._spare = self.key, self.value
        self.key, self.value = key, value
        self._swapped = not self._swapped
        self.frames -= evicted_frames

    def clear(self) -> None:
        """Forget the visual history but keep both arenas (and their addresses, which the
        captured step graphs of a stream refer to); the first arena becomes the live one again."""
        if self._swapped:
            (self.key, self.value), self._spare = self._spare, (self.key, self.value)
            self._swapped = False
        self.frames = 0

    def update_text(self, key: torch.Tensor, value: torch.Tensor) -> None:
        self.key[:, : self.text_tokens].copy_(key)
        self.value[:, : self.text_tokens].copy_(value)
