"""FIFO eviction + RoPE re-rotation of a streaming K/V cache.

Parity: reference ``wm/kernels/stream_cache.py:16-90`` (a Triton kernel there; a CUDA kernel
in ``csrc/stream_cache.cu`` here, PyTorch elsewhere).
"""

from __future__ import annotations

import torch

from agentgarten_b200.ops import native, reference

__all__ = ["relocate"]


def relocate(source: torch.Tensor, out: torch.Tensor, kept_tokens: int, shift_tokens: int,
             rotation: tuple[torch.Tensor, torch.Tensor] | None = None) -> None:
    """``out[:, r] = source[:, r]`` for ``r < kept_tokens`` and
    ``rotate(source[:, r + shift_tokens])`` behind it, for the ``source.shape[1] - shift_tokens``
    rows that survive.  ``source`` / ``out`` are ``[1, N, H, D]``; ``rotation`` is a pair of
    FP32 ``[1, N - shift_tokens, D]`` tables (``None``: plain move)."""
    destination, kept_prefix, shift = out, kept_tokens, shift_tokens
    kept = source.shape[1] - shift
    if (native.use(source) and source.shape[-1] == 128 and source.shape[0] == 1
            and source[0].is_contiguous() and destination[0].is_contiguous()):
        cos = sin = None
        if rotation is not None:
            cos = rotation[0].reshape(-1, 128).float().contiguous()
            sin = rotation[1].reshape(-1, 128).float().contiguous()
        native.ext().relocate(source[0], destination[0], kept, kept_prefix, shift, cos, sin)
        native.count()
        return
    cos = sin = None
    if rotation is not None:
        cos = rotation[0].reshape(-1, rotation[0].shape[-1])[kept_prefix:kept].float()
        sin = rotation[1].reshape(-1, rotation[1].shape[-1])[kept_prefix:kept].float()
    moved = reference.relocate_rows(source[0], kept_prefix, shift, kept, cos, sin)
    destination[0, :kept].copy_(moved[:kept])
