"""Adversarial Forcing: few-step distillation of a block-causal student (DMD + GAN).

Roles: a trainable few-step ``student``, a frozen teacher ``real_score``, a trainable
``fake_score`` that tracks the student's distribution, and optionally a ``discriminator``
head on the teacher's hidden features.  :class:`PhaseClock` decides the role of each
iteration: discriminator-only warm-up, then one student update every
``fake_score_updates_per_student + 1`` iterations, the rest train the fake score (and the
discriminator).

A student iteration is *Self Gradient Forcing*: pass 1 rolls the student out block by block
with its KV cache under ``no_grad`` up to a random exit step shared by all ranks; pass 2
replays the recorded queries through ``forward_ar`` with gradients (bitwise equal to pass 1,
see ``metrics/student/sgf_recovery_max_abs``) and receives the distribution-matching
gradient ``(x0_fake - x0_real) / mean|x0 - x0_real|`` computed in FP64, plus the generator
gradient of the GAN term.  The discriminator is regularised by finite-difference R1/R2 or
by the exact penalties of :mod:`agentgarten_b200.models.exact_regularization`.

Parity: reference ``wm/models/dmd.py:55-698``.
"""

from __future__ import annotations

import itertools
from collections.abc import Iterator, Mapping, Sequence
from dataclasses import dataclass, replace
from enum import StrEnum
from functools import partial
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from agentgarten_b200.infra.config import instantiate
from agentgarten_b200.infra.model import StepOutput, TrainingClosureSpec
from agentgarten_b200.infra.rng_state import isolated_rng
from agentgarten_b200.parallel.engine import ParallelConfig, parallelize_network
from agentgarten_b200.protocols import HistoryWindow
from agentgarten_b200.utils import log
from agentgarten_b200.utils.misc import frozen_parameters

from .base import ConditionedModel
from .exact_regularization import check_exact_regularization, exact_penalties
from .flow import UniformShift, invariant_randn, rf_interpolate, rf_x0, sampling_seeds

__all__ = ["RCM_ENDPOINTS", "DMDModel", "GANConfig", "PhaseClock", "Regularization"]

# Sigma endpoints of the 4-step rollout; an n-step rollout uses the first n.
RCM_ENDPOINTS = (1600.0 / 1601.0, 15.0 / 16.0, 5.0 / 6.0, 5.0 / 8.0)


class Regularization(StrEnum):
    FINITE_DIFFERENCE = "finite_difference"
    EXACT = "exact"


@dataclass(frozen=True)
class GANConfig:
    generator_weight: float = 0.01
    discriminator_weight: float = 0.01
    relativistic: bool = True
    regularization: Regularization = Regularization.FINITE_DIFFERENCE
    # finite difference: weight * E[(D(x + sigma*eps) - D(x))^2]
    regularization_weight: float = 30.0
    regularization_sigma: float = 0.05
    # exact: weight * E[||grad_x D||^2]; 0.075 = 30 * 0.05^2 matches the local scale above
    exact_regularization_weight: float = 0.075
    warmup_updates: int = 0

    def __post_init__(self) -> None:
        object.__setattr__(self, "regularization", Regularization(self.regularization))
        if self.warmup_updates < 0:
            raise ValueError("warmup_updates must be non-negative")


@dataclass(frozen=True)
class PhaseClock:
    fake_score_updates_per_student: int = 5
    warmup_updates: int = 0

    def __post_init__(self) -> None:
        if self.fake_score_updates_per_student < 1 or self.warmup_updates < 0:
            raise ValueError(f"invalid phase clock {self}")

    @property
    def cycle(self) -> int:
        return self.fake_score_updates_per_student + 1

    def is_warmup(self, iteration: int) -> bool:
        return iteration < self.warmup_updates

    def is_student(self, iteration: int) -> bool:
        return not self.is_warmup(iteration) and (iteration - self.warmup_updates) % self.cycle == 0

    def role_updates(self, iteration: int) -> dict[str, int]:
        """Updates each role has received after ``iteration`` iterations."""
        after_warmup = max(0, iteration - self.warmup_updates)
        student = -(-after_warmup // self.cycle)
        return {"student": student, "fake_score": after_warmup - student}

    def is_cadence_due(self, iteration: int, interval: int | None) -> bool:
        """Cadences count student updates and fire only at the end of a full cycle."""
        if interval is None or interval <= 0 or iteration <= 0:
            return False
        n = self.role_updates(iteration)
        return (n["student"] > 0 and n["student"] % interval == 0 and n["fake_score"] > 0
                and n["fake_score"] % (interval * self.fake_score_updates_per_student) == 0)


@dataclass
class _Rollout:
    noisy: Tensor   # [B, C, T, H, W] query of every block at its exit step
    sigma: Tensor   # [B, T]
    clean: Tensor   # [B, C, T, H, W] committed x0 (the generated clip)


def _pair_loss(real: Tensor, fake: Tensor, *, relativistic: bool) -> Tensor:
    if relativistic:
        return F.softplus(-(real - fake)).mean()
    return (F.softplus(-real) + F.softplus(fake)).mean()


def _pair_metrics(pair: Tensor, real: Tensor, fake: Tensor) -> dict[str, Tensor]:
    return {"metrics/discriminator/pair_loss": pair.detach(),
            "metrics/discriminator/accuracy": (real > fake).float().mean().detach()}


class DMDModel(ConditionedModel):
    checkpoint_excluded_prefixes = ("real_score.", "conditioner.")

    def __init__(self, *, student: nn.Module, real_score: nn.Module, fake_score: nn.Module,
                 conditioner: nn.Module, discriminator: Any = None, gan: GANConfig | None = None,
                 block_frames: int = 4, rollout_endpoints: Sequence[float] = RCM_ENDPOINTS,
                 score_shift: float = 5.0, real_score_guidance: float = 6.0,
                 fake_score_updates_per_student: int = 5, dmd_loss_scale: float = 0.5,
                 history: HistoryWindow | None = None,
                 student_trainable_patterns: Sequence[str] | None = None,
                 fake_score_trainable_patterns: Sequence[str] | None = None,
                 student_parallel: ParallelConfig | None = None,
                 score_parallel: ParallelConfig | None = None,
                 real_score_parallel: ParallelConfig | None = None,
                 discriminator_parallel: ParallelConfig | None = None,
                 conditioner_parallel: ParallelConfig | None = None,
                 sampling: Mapping[str, Any] | None = None, seed: int = 0) -> None:
        if (discriminator is None) != (gan is None):
            raise ValueError("pass both discriminator and gan, or neither")
        endpoints = tuple(float(v) for v in rollout_endpoints)
        if (not endpoints or any(not 0 < v <= 1 for v in endpoints)
                or any(a <= b for a, b in itertools.pairwise(endpoints))):
            raise ValueError(f"rollout endpoints must be strictly descending in (0, 1]: {endpoints}")
        if block_frames < 1 or int(block_frames) != block_frames:
            raise ValueError(f"block_frames must be a positive integer, got {block_frames}")
        super().__init__(conditioner=conditioner,
                         sampling_defaults={"num_steps": len(endpoints), "seed": 0},
                         sampling=sampling)
        self.student, self.real_score, self.fake_score = student, real_score, fake_score
        self.discriminator, self.gan = discriminator, gan
        self.block_frames = int(block_frames)
        self.rollout_endpoints = endpoints
        self.score_time = UniformShift(score_shift)
        self.real_score_guidance = float(real_score_guidance)
        self.clock = PhaseClock(fake_score_updates_per_student, gan.warmup_updates if gan else 0)
        self.dmd_loss_scale = float(dmd_loss_scale)
        self.history = history or HistoryWindow()
        plain = ParallelConfig(fully_shard=False, compile=False)
        self.student_parallel = student_parallel or plain
        self.score_parallel = score_parallel or plain
        self.real_score_parallel = real_score_parallel or self.score_parallel
        self.discriminator_parallel = discriminator_parallel or plain
        self.conditioner_parallel = conditioner_parallel or self.score_parallel
        self.seed = int(seed)
        self.real_score.requires_grad_(False)
        self.configure_trainable_parameters(student_trainable_patterns, module=self.student)
        self.configure_trainable_parameters(fake_score_trainable_patterns, module=self.fake_score)
        if gan is not None and gan.regularization is Regularization.EXACT:
            if self.real_score_parallel.context_parallel_size > 1:
                raise ValueError("exact R1/R2 does not support context parallelism: its "
                                 "forward-mode pass cannot cross the CP exchange. Use "
                                 "context_parallel_size=1 or finite_difference regularization")
            check_exact_regularization(self.real_score, discriminator)

    # ------------------------------------------------------------------- lifecycle
    def parallelize(self, device) -> None:
        mesh = parallelize_network(self.student, replace(self.student_parallel,
                                                         reshard_after_forward=False), device)
        others = [parallelize_network(self.real_score, self.real_score_parallel, device),
                  parallelize_network(self.fake_score, self.score_parallel, device)]
        self.parallelize_conditioner(self.conditioner_parallel, device)
        if self.discriminator is not None:
            self.discriminator.parallelize(self.discriminator_parallel, device)
        self.real_score.eval()
        self.register_context_parallel_mesh(mesh, *others)

    def train(self, mode: bool = True) -> "DMDModel":
        super().train(mode)
        self.real_score.eval()
        return self

    def is_cadence_due(self, iteration: int, interval: int | None) -> bool:
        return self.clock.is_cadence_due(int(iteration), interval)

    def get_optimizer_names(self, iteration: int) -> tuple[str, ...]:
        if self.clock.is_warmup(iteration):
            return ("discriminator",)
        if self.clock.is_student(iteration):
            return ("student",)
        return ("fake_score", "discriminator") if self.gan else ("fake_score",)

    def init_optimizer_scheduler(self, optimizer_config, scheduler_config):
        roles = {"student": self.student, "fake_score": self.fake_score}
        if self.discriminator is not None:
            roles["discriminator"] = self.discriminator
        missing = set(roles) - set(optimizer_config)
        if missing:
            raise KeyError(f"optimizer config lacks roles {sorted(missing)}")
        self.optimizer_dict, self.scheduler_dict = {}, {}
        for name, module in roles.items():
            optimizer = instantiate(optimizer_config[name],
                                    params=self._group_module_trainable_parameters(module))
            self.optimizer_dict[name] = optimizer
            self.scheduler_dict[name] = instantiate(scheduler_config, optimizer=optimizer)
        return self.optimizer_dict, self.scheduler_dict

    # --------------------------------------------------------------------- rollout
    def _exit_step(self, iteration: int) -> int:
        """Same draw on every rank: a CPU generator seeded from (seed, iteration)."""
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + iteration)
        return int(torch.randint(len(self.rollout_endpoints), (1,), generator=g))

    def _validate_rollout(self, frames: int, steps: int) -> None:
        if frames < 1 or frames % self.block_frames:
            raise ValueError("target latent frames must be a positive multiple of "
                             f"block_frames={self.block_frames}, got {frames}")
        if int(steps) != steps or not 1 <= steps <= len(self.rollout_endpoints):
            raise ValueError(f"num_steps must be an integer in [1, {len(self.rollout_endpoints)}], "
                             f"got {steps}")

    @torch.no_grad()
    def _rollout(self, anchor: Tensor, condition, frames: int, steps: int, *,
                 noise: Tensor | None = None) -> _Rollout:
        """``noise``: optional ``[steps, B, C, frames, H, W]`` draws; default global RNG."""
        self._validate_rollout(frames, steps)
        endpoints = self.rollout_endpoints[:steps]
        batch, device = anchor.shape[0], anchor.device
        shape = (batch, anchor.shape[1], self.block_frames, *anchor.shape[3:])
        cache = self.student.prefill(anchor, condition, history=self.history)
        queries, cleans = [], []
        clean = anchor
        blocks = frames // self.block_frames

        def draw(step: int, start: int) -> Tensor:
            if noise is None:
                return torch.randn(shape, device=device)
            return noise[step, :, :, start:start + self.block_frames]

        for index in range(blocks):
            start = index * self.block_frames
            current = draw(0, start)
            for step, sigma in enumerate(endpoints):
                level = torch.full((batch,), sigma, device=device)
                if step:
                    current = rf_interpolate(clean, draw(step, start), level)
                velocity = self.student.denoise(cache, current, level).float()
                clean = rf_x0(current, level, velocity)
            queries.append(current)
            cleans.append(clean)
            if index < blocks - 1:
                cache = self.student.commit(cache, clean)
        exit_sigma = torch.full((batch, frames), endpoints[-1], device=device)
        return _Rollout(torch.cat(queries, 2), exit_sigma, torch.cat(cleans, 2))

    # ---------------------------------------------------------------------- scores
    def _score(self, network, anchor, noisy, sigma, condition) -> Tensor:
        velocity = network(torch.cat((anchor, noisy), dim=2), sigma, condition, known_frames=1)
        return velocity[:, :, 1:].float()

    def _gan_roles(self):
        if self.gan is None or self.discriminator is None:
            raise RuntimeError("this objective was built without a discriminator")
        return self.gan, self.discriminator

    def _real_features(self, anchor, noisy, sigma, condition):
        """Hidden states of the frozen teacher at the discriminator's layers."""
        _, discriminator = self._gan_roles()
        _, features = self.real_score(torch.cat((anchor, noisy), dim=2), sigma, condition,
                                      known_frames=1, feature_layers=discriminator.feature_layers)
        return features

    def _real_velocity(self, anchor, noisy, sigma, conditions) -> Tensor:
        cond = self._score(self.real_score, anchor, noisy, sigma, conditions[0])
        if len(conditions) == 1:
            return cond
        uncond = self._score(self.real_score, anchor, noisy, sigma, conditions[1])
        return uncond + self.real_score_guidance * (cond - uncond)

    # -------------------------------------------------------------------- closures
    def training_step_closures(self, data_batch: dict[str, Any], iteration: int,
                               ) -> Iterator[TrainingClosureSpec]:
        latent = data_batch["latent"].float()
        anchor, real = latent[:, :, :1], latent[:, :, 1:]
        condition = self.conditioner.condition(data_batch)
        rollout = self._rollout(anchor, condition, real.shape[2], self._exit_step(iteration) + 1)
        if self.clock.is_student(iteration):
            conditions = [condition]
            if self.real_score_guidance != 1.0:
                conditions.append(self.conditioner.condition(data_batch, negative=True))
            yield "student", partial(self._student_loss, anchor, real, rollout, conditions), True
        else:
            yield ("fake_score",
                   partial(self._fake_score_loss, anchor, real, rollout.clean, condition,
                           warmup=self.clock.is_warmup(iteration)), True)

    def training_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        outputs, losses = {}, []
        for _name, closure, _last in self.training_step_closures(data_batch, iteration):
            out, loss = closure()
            outputs.update(out)
            losses.append(loss)
        return outputs, torch.stack(losses).sum()

    def _student_loss(self, anchor, real, rollout: _Rollout, conditions) -> StepOutput:
        velocity = self.student.forward_ar(
            anchor, rollout.noisy, rollout.sigma, conditions[0], block_frames=self.block_frames,
            clean=rollout.clean, history=self.history).float()
        x0 = rf_x0(rollout.noisy, rollout.sigma, velocity)
        target, gan_gradient, metrics = self._student_targets(anchor, real, x0.detach(), conditions)
        dmd = self.dmd_loss_scale * (x0.double() - target.double()).square().sum() / x0.numel()
        loss = dmd.float()
        if gan_gradient is not None:
            loss = loss + (x0 * gan_gradient).sum()  # injects dL_gan/dx0 as a linear term
        with torch.no_grad():
            recovery = (x0 - rollout.clean).abs().max()
        return {**metrics, "metrics/student/dmd_loss": dmd.detach(),
                "metrics/student/sgf_recovery_max_abs": recovery,
                "metrics/student/exit_sigma": rollout.sigma[0, 0]}, loss

    def _student_targets(self, anchor, real, x0, conditions):
        batch = x0.shape[0]
        sigma = self.score_time.sample(batch, device=x0.device)
        noise = torch.randn_like(x0)
        with torch.no_grad():
            noisy = rf_interpolate(x0, noise, sigma)
            fake_v = self._score(self.fake_score, anchor, noisy, sigma, conditions[0])
            real_v = self._real_velocity(anchor, noisy, sigma, conditions)
            x0_fake = rf_x0(noisy, sigma, fake_v).double()
            x0_real = rf_x0(noisy, sigma, real_v).double()
            scale = (x0.double() - x0_real).abs().flatten(1).mean(1).clamp_min(1e-5)
            gradient = (x0_fake - x0_real) / scale.view(-1, 1, 1, 1, 1)
            target = x0.double() - gradient
        gan_gradient, metrics = None, {}
        if self.gan is not None:
            gan_gradient, metrics = self._generator_gradient(anchor, real, x0, noise, sigma,
                                                             conditions[0])
        metrics["metrics/student/dmd_gradient_rms"] = gradient.float().square().mean().sqrt()
        return target, gan_gradient, metrics

    def _generator_gradient(self, anchor, real, x0, noise, sigma, condition):
        gan, discriminator = self._gan_roles()
        leaf = x0.detach().requires_grad_(True)
        # the head stays frozen for forward, backward and any recompute of this block
        with torch.enable_grad(), frozen_parameters(discriminator):
            fake_logits = discriminator([self._real_features(
                anchor, rf_interpolate(leaf, noise, sigma), sigma, condition)])
            with torch.no_grad():
                real_logits = discriminator([self._real_features(
                    anchor, rf_interpolate(real, noise, sigma), sigma, condition)])
            margin = fake_logits - real_logits if gan.relativistic else fake_logits
            loss = gan.generator_weight * F.softplus(-margin).mean()
            (gradient,) = torch.autograd.grad(loss, leaf)
        return torch.nan_to_num(gradient.detach()), {
            "metrics/student/gan_loss": loss.detach(),
            "metrics/student/gan_fake_minus_real_logit": margin.detach().mean()}

    def _fake_score_loss(self, anchor, real, generated, condition, *, warmup: bool) -> StepOutput:
        batch = generated.shape[0]
        sigma = self.score_time.sample(batch, device=generated.device)
        noise = torch.randn_like(generated)
        noisy = rf_interpolate(generated, noise, sigma)
        with torch.set_grad_enabled(torch.is_grad_enabled() and not warmup):
            velocity = self._score(self.fake_score, anchor, noisy, sigma, condition)
        fake_loss = (velocity - (noise - generated)).square().mean()
        outputs = {"metrics/fake_score/loss": fake_loss.detach()}
        loss = fake_loss if not warmup else fake_loss.detach() * 0
        if self.gan is not None:
            gan_loss, gan_metrics = self._discriminator_loss(anchor, real, noisy, noise, sigma,
                                                             condition)
            loss = loss + gan_loss
            outputs.update(gan_metrics)
        return outputs, loss

    def _discriminator_loss(self, anchor, real, fake_noisy, noise, sigma, condition):
        gan, discriminator = self._gan_roles()
        real_noisy = rf_interpolate(real, noise, sigma)
        if gan.regularization is Regularization.EXACT:
            return self._exact_discriminator_loss(anchor, real_noisy, fake_noisy, sigma, condition)
        rows = [fake_noisy, real_noisy]
        if gan.regularization_weight > 0:
            jitter = gan.regularization_sigma
            rows += [real_noisy + jitter * torch.randn_like(real_noisy),
                     fake_noisy + jitter * torch.randn_like(fake_noisy)]
        n = len(rows)
        with torch.no_grad():
            features = self._real_features(torch.cat((anchor,) * n), torch.cat(rows),
                                           sigma.repeat(n), condition.repeat(n))
        logits = discriminator([features]).split(fake_noisy.shape[0])
        fake_logits, real_logits = logits[0], logits[1]
        pair = _pair_loss(real_logits, fake_logits, relativistic=gan.relativistic)
        loss = gan.discriminator_weight * pair
        metrics = _pair_metrics(pair, real_logits, fake_logits)
        if gan.regularization_weight > 0:
            r1 = (logits[2] - real_logits).square().mean()
            r2 = (logits[3] - fake_logits).square().mean()
            loss = loss + gan.discriminator_weight * 0.5 * gan.regularization_weight * (r1 + r2)
            metrics.update({"metrics/discriminator/r1": r1.detach(),
                            "metrics/discriminator/r2": r2.detach()})
        return loss, metrics

    def _exact_discriminator_loss(self, anchor, real_noisy, fake_noisy, sigma, condition):
        gan, discriminator = self._gan_roles()
        batch = fake_noisy.shape[0]
        features = partial(self._real_features, torch.cat((anchor, anchor)),
                           sigma=sigma.repeat(2), condition=condition.repeat(2))
        result = exact_penalties(features, discriminator, torch.cat((fake_noisy, real_noisy)))
        fake_logits, real_logits = result.logits.split(batch)
        pair = _pair_loss(real_logits, fake_logits, relativistic=gan.relativistic)
        r2, r1 = result.penalty.split(batch)
        scale = gan.discriminator_weight * 0.5 * gan.exact_regularization_weight
        # value: weighted R1 + R2; gradient: the exact dR/dtheta carried by the surrogate
        regular = scale * ((r1.mean() + r2.mean()) + result.surrogate.view(2, batch).mean(1).sum())
        return gan.discriminator_weight * pair + regular, {
            **_pair_metrics(pair, real_logits, fake_logits),
            "metrics/discriminator/r1": r1.mean(), "metrics/discriminator/r2": r2.mean()}

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def validation_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        del iteration
        latent = data_batch["latent"].float()
        anchor, real = latent[:, :, :1], latent[:, :, 1:]
        condition = self.conditioner.condition(data_batch)
        with isolated_rng():  # fixed seed for every validation batch, caller's streams untouched
            torch.manual_seed(self.seed)
            rollout = self._rollout(anchor, condition, real.shape[2], len(self.rollout_endpoints))
            return self._fake_score_loss(anchor, real, rollout.clean, condition, warmup=False)

    @torch.inference_mode()
    def sample(self, data_batch: dict[str, Any], **options: Any) -> dict[str, Tensor]:
        options = self.sampling_options(options)
        latent = data_batch["latent"].float()
        anchor, target = latent[:, :, :1], latent[:, :, 1:]
        self._validate_rollout(target.shape[2], options["num_steps"])
        steps = int(options["num_steps"])
        seeds = sampling_seeds(data_batch, int(options["seed"]))
        noise = torch.stack([invariant_randn(target, seeds, stream=s) for s in range(steps)])
        rollout = self._rollout(anchor, self.conditioner.condition(data_batch), target.shape[2],
                                steps, noise=noise)
        return {**self.conditioner.visuals(data_batch),
                "ground_truth": self.conditioner.decode(latent),
                "sample": self.conditioner.decode(torch.cat((anchor, rollout.clean), dim=2))}
