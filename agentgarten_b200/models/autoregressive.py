"""Block-causal autoregressive objective with teacher forcing or diffusion forcing.

The clip is an anchor frame plus blocks of ``block_frames`` frames; every block draws its
own sigma.  *Teacher forcing* gives each noisy block the clean earlier blocks as history
(optionally corrupted per frame — exposure change, additive noise or a down/up rescale — so
the model tolerates its own imperfect history at inference).  *Diffusion forcing* uses the
noisy blocks themselves as history.  Sampling prefills a KV cache with the anchor, then per
block runs UniPC over ``denoise`` and ``commit``s the result.

Parity: reference ``wm/models/autoregressive.py:29-243``.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from enum import StrEnum
from functools import partial
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


_EXPOSURE = (0.3, 1.7)       # contrast around the per-pixel channel mean
_NOISE = (0.0, 1.0 / 3.0)    # blend weight of Gaussian noise
_RESCALE = (0.9, 1.0)        # bilinear down-then-up factor


@torch.no_grad()
def corrupt_history(frames: torch.Tensor, generator: torch.Generator | None = None) -> torch.Tensor:
    """Per frame, one of: exposure change, noise blend, rescale blur, or nothing."""
    b, _, t, h, w = frames.shape
    device = frames.device
    kind = torch.randint(4, (b, t), device=device, generator=generator)
    u = torch.rand(b, t, device=device, generator=generator)

    def within(lo_hi):
        return lo_hi[0] + u * (lo_hi[1] - lo_hi[0])

    amount = torch.where(kind == 0, within(_EXPOSURE),
                         torch.where(kind == 1, within(_NOISE), within(_RESCALE)))
    amount5, kind5 = amount[:, None, :, None, None], kind[:, None, :, None, None]
    mean = frames.mean(dim=1, keepdim=True)
    noise = torch.randn(frames.shape, device=device, generator=generator)
    out = torch.where(kind5 == 0, (frames - mean) * amount5 + mean, frames)
    out = torch.where(kind5 == 1, amount5 * noise + (1.0 - amount5) * frames, out)
    for bi, ti in (kind == 2).nonzero().tolist():
        s = float(amount[bi, ti])
        small = (max(1, round(h * s)), max(1, round(w * s)))
        frame = frames[bi:bi + 1, :, ti]
        down = F.interpolate(frame, size=small, mode="bilinear", antialias=True)
        out[bi:bi + 1, :, ti] = F.interpolate(down, size=(h, w), mode="bilinear", antialias=True)
    return out


class AutoregressiveModel(ConditionedModel):
    def __init__(self, *, net: nn.Module, conditioner: nn.Module,
                 mode: ARMode | str = ARMode.TEACHER_FORCING, block_frames: int = 4,
                 schedule: RectifiedFlowSchedule | None = None, text_dropout: float = 0.1,
                 corrupt_clean_history: bool = True, diffusion_forcing_clean_sigma: float = 0.001,
                 trainable_patterns: Sequence[str] | None = None,
                 parallel: ParallelConfig | None = None,
                 conditioner_parallel: ParallelConfig | None = None,
                 sampling: Mapping[str, Any] | None = None, validation_seed: int = 0) -> None:
        super().__init__(conditioner=conditioner,
                         sampling_defaults={"num_steps": 16, "guidance": 6.0, "seed": 0,
                                            "sink_blocks": 0, "recent_blocks": None},
                         sampling=sampling)
        self.net = net
        self.mode = ARMode(mode)
        self.block_frames = int(block_frames)
        self.schedule = schedule or RectifiedFlowSchedule(shift=5.0, train_distribution="waver")
        self.text_dropout = float(text_dropout)
        self.corrupt_clean_history = bool(corrupt_clean_history)
        self.diffusion_forcing_clean_sigma = float(diffusion_forcing_clean_sigma)
        self.parallel = parallel or ParallelConfig(fully_shard=False, compile=False)
        self.conditioner_parallel = conditioner_parallel or self.parallel
        self.validation_seed = int(validation_seed)
        self.configure_trainable_parameters(trainable_patterns, module=self.net)

    def parallelize(self, device) -> None:
        mesh = parallelize_network(self.net, self.parallel, device)
        self.parallelize_conditioner(self.conditioner_parallel, device)
        self.register_context_parallel_mesh(mesh)

    # ------------------------------------------------------------------- training
    def _block_sigma(self, batch: int, frames: int, device, generator) -> torch.Tensor:
        per_block = self.schedule.sample((batch, frames // self.block_frames), device=device,
                                         generator=generator)
        return per_block.repeat_interleave(self.block_frames, dim=1)

    def _loss(self, batch: Mapping[str, Any], *, generator, training: bool) -> StepOutput:
        latent = batch["latent"].float()
        anchor, target = latent[:, :, :1], latent[:, :, 1:]
        count, _, frames = target.shape[:3]
        if frames % self.block_frames:
            raise ValueError(f"{frames} target frames are not a multiple of {self.block_frames}")
        device = latent.device
        sigma = self._block_sigma(count, frames, device, generator)
        noise = torch.randn(target.shape, device=device, generator=generator)
        noisy = rf_interpolate(target, noise, sigma)
        clean = None
        if self.mode is ARMode.TEACHER_FORCING:
            clean = corrupt_history(target, generator) if training and self.corrupt_clean_history \
                else target
        drop = None
        if training:
            drop = torch.rand(count, device=device, generator=generator) < self.text_dropout
        condition = self.conditioner.condition(batch, drop=drop)
        velocity = self.net.forward_ar(anchor, noisy, sigma, condition,
                                       block_frames=self.block_frames, clean=clean).float()
        per_sample = (velocity - (noise - target)).square().flatten(1).mean(1)
        return {"loss_per_sample": per_sample.detach(), "sigma": sigma.detach()}, per_sample.mean()

    def training_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        del iteration
        return self._loss(data_batch, generator=None, training=True)

    @torch.no_grad()
    def validation_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        del iteration
        generator = torch.Generator(device=data_batch["latent"].device)
        generator.manual_seed(self.validation_seed)
        return self._loss(data_batch, generator=generator, training=False)

    # ------------------------------------------------------------------- sampling
    def _guided(self, caches: Sequence[Any], guidance: float, current: torch.Tensor,
                sigma: float) -> torch.Tensor:
        """``caches`` = (conditional[, negative]); classifier-free guidance when both exist."""
        per_sample = torch.full((current.shape[0],), sigma, device=current.device)
        outs = [self.net.denoise(c, current, per_sample).float() for c in caches]
        return outs[0] if len(outs) == 1 else outs[1] + guidance * (outs[0] - outs[1])

    @torch.inference_mode()
    def sample(self, data_batch: dict[str, Any], **options: Any) -> dict[str, torch.Tensor]:
        options = self.sampling_options(options)
        latent = data_batch["latent"].float()
        window = HistoryWindow(int(options["sink_blocks"]), options["recent_blocks"])
        guidance = float(options["guidance"])
        conditions = [self.conditioner.condition(data_batch)]
        if guidance != 1.0:
            conditions.append(self.conditioner.condition(data_batch, negative=True))
        anchor = latent[:, :, :1]
        caches = [self.net.prefill(anchor, c, history=window) for c in conditions]
        noise = invariant_randn(latent[:, :, 1:], sampling_seeds(data_batch, int(options["seed"])))
        commit_sigma = None
        if self.mode is ARMode.DIFFUSION_FORCING:
            commit_sigma = torch.full((latent.shape[0],), self.diffusion_forcing_clean_sigma,
                                      device=latent.device)
        solver = FlowUniPC(int(options["num_steps"]), shift=self.schedule.shift)
        blocks = []
        for start in range(0, noise.shape[2], self.block_frames):
            block = solver.run(noise[:, :, start:start + self.block_frames].clone(),
                               partial(self._guided, caches, guidance))
            caches = [self.net.commit(c, block, commit_sigma) for c in caches]
            blocks.append(block)
        generated = torch.cat((anchor, *blocks), dim=2)
        return {**self.conditioner.visuals(data_batch),
                "ground_truth": self.conditioner.decode(latent),
                "sample": self.conditioner.decode(generated)}
