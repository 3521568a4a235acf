"""FIFO eviction + RoPE re-rotation of a streaming K/V cache.

Parity: reference ``wm/kernels/stream_cache.py:16-90`` (a Triton kernel there; a CUDA kernel
in ``csrc/stream_cache.cu`` here, PyTorch elsewhere).
"""

from __future__ import annotations

import torch

from agentgarten_b200.ops import native, reference

__all__ = ["relocate"]


def relocate(source: torch.Tensor, destination: torch.Tensor, kept_prefix: int, shift: int,
             rotation: tuple[torch.Tensor, torch.Tensor] | None = None) -> None:
    """``destination[:, r] = source[:, r]`` for ``r < kept_prefix`` and
    ``rotate(source[:, r + shift])`` behind it, for the ``source.shape[1] - shift`` rows
    that survive.  ``source``/``destination`` are ``[1, N, H, D]``; ``rotation`` is a pair of
    FP32 ``[1, N - shift, D]`` tables (``None``: plain move)."""
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
