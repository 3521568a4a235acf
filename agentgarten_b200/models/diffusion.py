"""Bidirectional rectified-flow objective.

A training example is a *draw*: one sigma per clip, Gaussian noise of the clip's shape, the
interpolated clip with its first ``known_frames`` frames put back clean (the anchor the
network may rely on), and the regression target ``noise - clean``.  The loss is the squared
velocity error over the frames that were actually corrupted, divided by the element count of
a whole clip, so clips with more known frames weigh less rather than more.  Random numbers
are consumed in a fixed order (sigma, noise, text dropout), which is what makes a seeded run
repeat the reference's loss sequence.

Sampling integrates the flow ODE with the UniPC solver; classifier-free guidance evaluates the
network on the prompt and on the negative prompt and extrapolates, and after every solver step
the known frames are restored.

Parity: reference ``wm/models/diffusion.py:26-148`` (constructor keywords, step outputs
``loss_per_sample`` / ``sigma``, sample outputs ``ground_truth`` / ``sample``).
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from agentgarten_b200.infra.model import StepOutput
from agentgarten_b200.parallel.engine import ParallelConfig, parallelize_network

from .base import ConditionedModel
from .flow import FlowUniPC, RectifiedFlowSchedule, invariant_randn, rf_interpolate, sampling_seeds

__all__ = ["DiffusionModel"]


@dataclass(frozen=True)
class _Draw:
    """One corrupted clip: network input, regression target and the noise level used."""

    noisy: torch.Tensor
    target: torch.Tensor
    sigma: torch.Tensor


class _GuidedVelocity:
    """Velocity field handed to the ODE solver: the network under one prompt, or the
    classifier-free extrapolation from the negative prompt towards the prompt."""

    def __init__(self, net: nn.Module, prompt, negative, scale: float, known: int, batch: int,
                 device: torch.device) -> None:
        self.net, self.prompt, self.negative = net, prompt, negative
        self.scale, self.known, self.batch, self.device = scale, known, batch, device

    def __call__(self, latent: torch.Tensor, sigma: float) -> torch.Tensor:
        level = torch.full((self.batch,), sigma, device=self.device)
        towards = self.net(latent, level, self.prompt, known_frames=self.known).float()
        if self.negative is None:
            return towards
        away = self.net(latent, level, self.negative, known_frames=self.known).float()
        return away + self.scale * (towards - away)


class DiffusionModel(ConditionedModel):
    def __init__(self, *, net: nn.Module, conditioner: nn.Module,
                 schedule: RectifiedFlowSchedule | None = None, known_frames: int = 1,
                 text_dropout: float = 0.1, trainable_patterns: Sequence[str] | None = None,
                 parallel: ParallelConfig | None = None,
                 conditioner_parallel: ParallelConfig | None = None,
                 sampling: Mapping[str, Any] | None = None, validation_seed: int = 0) -> None:
        if not 0.0 <= text_dropout <= 1.0:
            raise ValueError(f"text_dropout must be in [0, 1], got {text_dropout}")
        super().__init__(conditioner=conditioner, sampling=sampling,
                         sampling_defaults={"num_steps": 35, "guidance": 6.0, "seed": 0})
        self.net = net
        self.schedule = schedule if schedule is not None else \
            RectifiedFlowSchedule(shift=5.0, train_distribution="waver")
        self.known_frames = int(known_frames)
        self.text_dropout = float(text_dropout)
        self.parallel = parallel if parallel is not None else ParallelConfig(fully_shard=False, compile=False)
        self.conditioner_parallel = conditioner_parallel if conditioner_parallel is not None else self.parallel
        self.validation_seed = int(validation_seed)
        self.configure_trainable_parameters(trainable_patterns, module=self.net)

    def parallelize(self, device) -> None:
        self.register_context_parallel_mesh(parallelize_network(self.net, self.parallel, device))
        self.parallelize_conditioner(self.conditioner_parallel, device)

    # ------------------------------------------------------------------- training
    def _draw(self, clean: torch.Tensor, generator: torch.Generator | None) -> _Draw:
        sigma = self.schedule.sample(clean.shape[0], device=clean.device, generator=generator)
        noise = torch.randn(clean.shape, device=clean.device, generator=generator)
        noisy = rf_interpolate(clean, noise, sigma)
        anchor = slice(0, self.known_frames)
        noisy[:, :, anchor] = clean[:, :, anchor]
        return _Draw(noisy=noisy, target=noise - clean, sigma=sigma)

    def _objective(self, batch: Mapping[str, Any], generator: torch.Generator | None,
                   dropout: float | None) -> StepOutput:
        clean = batch["latent"].float()
        draw = self._draw(clean, generator)
        dropped = None
        if dropout is not None:
            coin = torch.rand(clean.shape[0], device=clean.device, generator=generator)
            dropped = coin < dropout
        condition = self.conditioner.condition(batch, drop=dropped)
        predicted = self.net(draw.noisy, draw.sigma, condition, known_frames=self.known_frames).float()
        residual = (predicted - draw.target)[:, :, self.known_frames:]
        per_clip = residual.square().flatten(1).sum(1) / clean[0].numel()
        report = {"loss_per_sample": per_clip.detach(), "sigma": draw.sigma.detach()}
        return report, per_clip.mean()

    def training_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        return self._objective(data_batch, None, self.text_dropout)

    @torch.no_grad()
    def validation_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        # one fixed seed: every validation round scores the same corruptions
        fixed = torch.Generator(device=data_batch["latent"].device).manual_seed(self.validation_seed)
        return self._objective(data_batch, fixed, None)

    # ------------------------------------------------------------------- sampling
    @torch.inference_mode()
    def sample(self, data_batch: dict[str, Any], **options: Any) -> dict[str, torch.Tensor]:
        chosen = self.sampling_options(options)
        clean = data_batch["latent"].float()
        anchor = slice(0, self.known_frames)
        scale = float(chosen["guidance"])
        field = _GuidedVelocity(
            self.net, self.conditioner.condition(data_batch),
            self.conditioner.condition(data_batch, negative=True) if scale != 1.0 else None,
            scale, self.known_frames, clean.shape[0], clean.device)

        def restore_anchor(latent: torch.Tensor) -> torch.Tensor:
            latent[:, :, anchor] = clean[:, :, anchor]
            return latent

        start = restore_anchor(invariant_randn(clean, sampling_seeds(data_batch, int(chosen["seed"]))))
        solver = FlowUniPC(int(chosen["num_steps"]), shift=self.schedule.shift)
        result = solver.run(start, field, post_step=restore_anchor)
        panels = dict(self.conditioner.visuals(data_batch))
        panels["ground_truth"] = self.conditioner.decode(clean)
        panels["sample"] = self.conditioner.decode(result)
        return panels
