"""Block-causal autoregressive objective (teacher forcing or diffusion forcing).

A clip is its first frame (the anchor, always clean) followed by blocks of ``block_frames``
frames.  Every block of every sample draws its own noise level; the network sees all blocks
in one block-causal pass (``forward_ar``) and is asked for the velocity of each noisy block.

* **Teacher forcing** — the history a block attends to is the *clean* earlier blocks.  During
  training that history is degraded frame by frame (a contrast change, a blend with noise, a
  down/up rescale, or nothing) so that the model learns to continue from its own imperfect
  output.
* **Diffusion forcing** — the history is the noisy blocks themselves, each at its own level.

Random numbers are drawn in a fixed order: block sigmas, noise, history degradation, text
dropout.  Sampling fills a KV cache with the anchor, then for each block integrates the flow
ODE against the cache and commits the finished block (under diffusion forcing at a small
positive sigma, as in training).

Parity: reference ``wm/models/autoregressive.py:29-243`` (constructor keywords, ``ARMode``,
``corrupt_history``, step and sample outputs).
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from enum import StrEnum
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

from agentgarten_b200.infra.model import StepOutput
from agentgarten_b200.parallel.engine import ParallelConfig, parallelize_network
from agentgarten_b200.protocols import HistoryWindow

from .base import ConditionedModel
from .flow import FlowUniPC, RectifiedFlowSchedule, invariant_randn, rf_interpolate, sampling_seeds

__all__ = ["ARMode", "AutoregressiveModel", "corrupt_history"]


class ARMode(StrEnum):
    TEACHER_FORCING = "teacher_forcing"
    DIFFUSION_FORCING = "diffusion_forcing"


# Degradations of a history frame, indexed by the drawn kind; each has a strength range from
# which one uniform number picks.  Kind 3 leaves the frame alone.
_CONTRAST, _NOISE_BLEND, _RESCALE, _UNTOUCHED = range(4)
_STRENGTH = {_CONTRAST: (0.3, 1.7), _NOISE_BLEND: (0.0, 1.0 / 3.0), _RESCALE: (0.9, 1.0)}


def _blur_by_rescale(frame: torch.Tensor, factor: float) -> torch.Tensor:
    """``frame`` [1, C, H, W] shrunk by ``factor`` and enlarged again (bilinear, antialiased)."""
    height, width = frame.shape[-2:]
    reduced = (max(1, round(height * factor)), max(1, round(width * factor)))
    small = F.interpolate(frame, size=reduced, mode="bilinear", antialias=True)
    return F.interpolate(small, size=(height, width), mode="bilinear", antialias=True)


@torch.no_grad()
def corrupt_history(frames: torch.Tensor, generator: torch.Generator | None = None) -> torch.Tensor:
    """Degrade every frame of ``frames`` [B, C, T, H, W] independently (see module text)."""
    samples, _, count = frames.shape[:3]
    device = frames.device
    kind = torch.randint(4, (samples, count), device=device, generator=generator)
    pick = torch.rand(samples, count, device=device, generator=generator)
    gaussian = torch.randn(frames.shape, device=device, generator=generator)

    strength = torch.zeros_like(pick)
    for which, (low, high) in _STRENGTH.items():
        strength = torch.where(kind == which, low + pick * (high - low), strength)
    per_frame = (slice(None), None, slice(None), None, None)  # [B, T] -> [B, 1, T, 1, 1]
    amount, chosen = strength[per_frame], kind[per_frame]

    centre = frames.mean(dim=1, keepdim=True)
    degraded = torch.where(chosen == _CONTRAST, centre + (frames - centre) * amount, frames)
    degraded = torch.where(chosen == _NOISE_BLEND, amount * gaussian + (1.0 - amount) * frames, degraded)
    for sample, index in torch.nonzero(kind == _RESCALE).tolist():
        degraded[sample:sample + 1, :, index] = _blur_by_rescale(
            frames[sample:sample + 1, :, index], float(strength[sample, index]))
    return degraded


class _CachedGuidance:
    """The KV caches of one sampling run (prompt, and negative prompt under guidance) and the
    guided velocity over them."""

    def __init__(self, net: nn.Module, caches: list[Any], scale: float) -> None:
        self.net, self.caches, self.scale = net, caches, scale

    def __call__(self, latent: torch.Tensor, sigma: float) -> torch.Tensor:
        level = torch.full((latent.shape[0],), sigma, device=latent.device)
        towards = self.net.denoise(self.caches[0], latent, level).float()
        if len(self.caches) == 1:
            return towards
        away = self.net.denoise(self.caches[1], latent, level).float()
        return away + self.scale * (towards - away)

    def publish(self, block: torch.Tensor, sigma: torch.Tensor | None) -> None:
        self.caches = [self.net.commit(cache, block, sigma) for cache in self.caches]


class AutoregressiveModel(ConditionedModel):
    def __init__(self, *, net: nn.Module, conditioner: nn.Module,
                 mode: ARMode | str = ARMode.TEACHER_FORCING, block_frames: int = 4,
                 schedule: RectifiedFlowSchedule | None = None, text_dropout: float = 0.1,
                 corrupt_clean_history: bool = True, diffusion_forcing_clean_sigma: float = 0.001,
                 trainable_patterns: Sequence[str] | None = None,
                 parallel: ParallelConfig | None = None,
                 conditioner_parallel: ParallelConfig | None = None,
                 sampling: Mapping[str, Any] | None = None, validation_seed: int = 0) -> None:
        defaults = {"num_steps": 16, "guidance": 6.0, "seed": 0, "sink_blocks": 0, "recent_blocks": None}
        super().__init__(conditioner=conditioner, sampling_defaults=defaults, sampling=sampling)
        self.net = net
        self.mode = ARMode(mode)
        self.block_frames = int(block_frames)
        self.schedule = schedule if schedule is not None else \
            RectifiedFlowSchedule(shift=5.0, train_distribution="waver")
        self.text_dropout = float(text_dropout)
        self.corrupt_clean_history = bool(corrupt_clean_history)
        self.diffusion_forcing_clean_sigma = float(diffusion_forcing_clean_sigma)
        self.parallel = parallel if parallel is not None else ParallelConfig(fully_shard=False, compile=False)
        self.conditioner_parallel = conditioner_parallel if conditioner_parallel is not None else self.parallel
        self.validation_seed = int(validation_seed)
        self.configure_trainable_parameters(trainable_patterns, module=self.net)

    def parallelize(self, device) -> None:
        self.register_context_parallel_mesh(parallelize_network(self.net, self.parallel, device))
        self.parallelize_conditioner(self.conditioner_parallel, device)

    # ------------------------------------------------------------------- training
    def _sigma_per_frame(self, samples: int, frames: int, device, generator) -> torch.Tensor:
        """One level per (sample, block), repeated over the frames of the block."""
        blocks, ragged = divmod(frames, self.block_frames)
        if ragged:
            raise ValueError(f"{frames} target frames are not a multiple of {self.block_frames}")
        levels = self.schedule.sample((samples, blocks), device=device, generator=generator)
        return levels.repeat_interleave(self.block_frames, dim=1)

    def _objective(self, batch: Mapping[str, Any], generator, training: bool) -> StepOutput:
        clip = batch["latent"].float()
        anchor, future = clip[:, :, :1], clip[:, :, 1:]
        samples, device = clip.shape[0], clip.device
        sigma = self._sigma_per_frame(samples, future.shape[2], device, generator)
        noise = torch.randn(future.shape, device=device, generator=generator)
        corrupted = rf_interpolate(future, noise, sigma)
        history = None
        if self.mode is ARMode.TEACHER_FORCING:
            degrade = training and self.corrupt_clean_history
            history = corrupt_history(future, generator) if degrade else future
        dropped = None
        if training:
            dropped = torch.rand(samples, device=device, generator=generator) < self.text_dropout
        condition = self.conditioner.condition(batch, drop=dropped)
        predicted = self.net.forward_ar(anchor, corrupted, sigma, condition,
                                        block_frames=self.block_frames, clean=history).float()
        per_clip = (predicted - (noise - future)).square().flatten(1).mean(1)
        return {"loss_per_sample": per_clip.detach(), "sigma": sigma.detach()}, per_clip.mean()

    def training_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        return self._objective(data_batch, None, True)

    @torch.no_grad()
    def validation_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        fixed = torch.Generator(device=data_batch["latent"].device).manual_seed(self.validation_seed)
        return self._objective(data_batch, fixed, False)

    # ------------------------------------------------------------------- sampling
    @torch.inference_mode()
    def sample(self, data_batch: dict[str, Any], **options: Any) -> dict[str, torch.Tensor]:
        chosen = self.sampling_options(options)
        clip = data_batch["latent"].float()
        anchor = clip[:, :, :1]
        scale = float(chosen["guidance"])
        window = HistoryWindow(int(chosen["sink_blocks"]), chosen["recent_blocks"])
        prompts = [self.conditioner.condition(data_batch)]
        if scale != 1.0:
            prompts.append(self.conditioner.condition(data_batch, negative=True))
        field = _CachedGuidance(
            self.net, [self.net.prefill(anchor, prompt, history=window) for prompt in prompts], scale)
        publish_at = None
        if self.mode is ARMode.DIFFUSION_FORCING:
            publish_at = clip.new_full((clip.shape[0],), self.diffusion_forcing_clean_sigma)
        start = invariant_randn(clip[:, :, 1:], sampling_seeds(data_batch, int(chosen["seed"])))
        solver = FlowUniPC(int(chosen["num_steps"]), shift=self.schedule.shift)
        pieces = [anchor]
        for first in range(0, start.shape[2], self.block_frames):
            finished = solver.run(start[:, :, first:first + self.block_frames].clone(), field)
            field.publish(finished, publish_at)
            pieces.append(finished)
        panels = dict(self.conditioner.visuals(data_batch))
        panels["ground_truth"] = self.conditioner.decode(clip)
        panels["sample"] = self.conditioner.decode(torch.cat(pieces, dim=2))
        return panels
