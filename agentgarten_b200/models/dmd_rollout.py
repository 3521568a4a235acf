"""Few-step rollout of the block-causal student through its KV cache.

Every block starts from pure noise at the first endpoint and is refined at the following
endpoints by re-noising the current clean estimate; the query of the block at its *last*
step is recorded, because the differentiable replay (``forward_ar`` over all recorded queries
with the committed clean blocks as history) must reproduce exactly that network evaluation.
Finished blocks are committed to the cache, except the last one, which nothing attends to.

Parity: reference ``wm/models/dmd.py:300-350``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch
from torch import Tensor, nn

from agentgarten_b200.protocols import HistoryWindow

from .flow import rf_interpolate, rf_x0

__all__ = ["Rollout", "StudentRollout"]


@dataclass
class Rollout:
    noisy: Tensor   # [B, C, T, H, W] what the student saw for each block at its exit step
    sigma: Tensor   # [B, T] the exit level, per frame
    clean: Tensor   # [B, C, T, H, W] the generated clip (committed estimates)


class _Noise:
    """Noise of (step, block): fresh draws from the global generator, or slices of a tensor
    ``[steps, B, C, T, H, W]`` prepared by the caller (seeded sampling)."""

    def __init__(self, shape: tuple[int, ...], device: torch.device, prepared: Tensor | None) -> None:
        self.shape, self.device, self.prepared = shape, device, prepared

    def __call__(self, step: int, first_frame: int) -> Tensor:
        if self.prepared is None:
            return torch.randn(self.shape, device=self.device)
        return self.prepared[step, :, :, first_frame:first_frame + self.shape[2]]


class StudentRollout:
    def __init__(self, student: nn.Module, endpoints: Sequence[float], block_frames: int,
                 history: HistoryWindow) -> None:
        self.student, self.endpoints = student, tuple(endpoints)
        self.block_frames, self.history = int(block_frames), history

    def check(self, frames: int, steps: int) -> None:
        if frames < 1 or frames % self.block_frames:
            raise ValueError("target latent frames must be a positive multiple of "
                             f"block_frames={self.block_frames}, got {frames}")
        if int(steps) != steps or not 1 <= steps <= len(self.endpoints):
            raise ValueError(f"num_steps must be an integer in [1, {len(self.endpoints)}], got {steps}")

    def _refine(self, cache, noise: _Noise, first_frame: int, levels, previous: Tensor):
        """One block through all its levels → (last query, clean estimate)."""
        batch, device = previous.shape[0], previous.device
        query = estimate = None
        for step, value in enumerate(levels):
            level = torch.full((batch,), value, device=device)
            drawn = noise(step, first_frame)
            query = drawn if step == 0 else rf_interpolate(estimate, drawn, level)
            estimate = rf_x0(query, level, self.student.denoise(cache, query, level).float())
        return query, estimate

    @torch.no_grad()
    def run(self, anchor: Tensor, condition, frames: int, steps: int, *,
            noise: Tensor | None = None) -> Rollout:
        self.check(frames, steps)
        levels = self.endpoints[:steps]
        block = self.block_frames
        source = _Noise((anchor.shape[0], anchor.shape[1], block, *anchor.shape[3:]), anchor.device, noise)
        cache = self.student.prefill(anchor, condition, history=self.history)
        queries, estimates = [], []
        for first_frame in range(0, frames, block):
            query, estimate = self._refine(cache, source, first_frame, levels, anchor)
            queries.append(query)
            estimates.append(estimate)
            if first_frame + block < frames:
                cache = self.student.commit(cache, estimate)
        exit_level = anchor.new_full((anchor.shape[0], frames), levels[-1], dtype=torch.float32)
        return Rollout(torch.cat(queries, dim=2), exit_level, torch.cat(estimates, dim=2))
