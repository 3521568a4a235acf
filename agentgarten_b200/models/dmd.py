"""Adversarial Forcing: few-step distillation of a block-causal student (DMD + GAN).

Four roles: the trainable few-step ``student``; the frozen teacher ``real_score``; the
trainable ``fake_score`` that follows the student's output distribution; optionally a
``discriminator`` head on the teacher's hidden features (:mod:`.dmd_adversarial`).  A
:class:`PhaseClock` gives each iteration its role: discriminator-only warm-up, then one
student update per cycle, the other iterations train the fake score and the discriminator.

Every iteration first rolls the student out without gradients (:mod:`.dmd_rollout`) up to an
exit step drawn identically on every rank.  On a student iteration the recorded queries are
replayed through ``forward_ar`` with gradients — bit for bit the same evaluation, which the
``metrics/student/sgf_recovery_max_abs`` output monitors — and the clean estimate receives

* the distribution-matching gradient ``(x0_fake - x0_real) / mean|x0 - x0_real|`` of the two
  score networks at a random noise level (FP64, injected as a squared distance to a detached
  target), and
* the generator gradient of the GAN term, injected as a linear term.

On the other iterations the fake score regresses the rectified-flow velocity of the generated
clip and the discriminator separates noised real clips from noised generated ones.

Parity: reference ``wm/models/dmd.py:55-698`` (roles, constructor keywords, optimizer role
names, metric names, checkpoint exclusions).
"""

from __future__ import annotations

import itertools
from collections.abc import Iterator, Mapping, Sequence
from dataclasses import replace
from typing import Any

import torch
from torch import Tensor, nn

from agentgarten_b200 import ops
from agentgarten_b200.infra.config import instantiate
from agentgarten_b200.infra.model import StepOutput, TrainingClosureSpec
from agentgarten_b200.infra.rng_state import isolated_rng
from agentgarten_b200.parallel.engine import ParallelConfig, parallelize_network
from agentgarten_b200.protocols import HistoryWindow

from .base import ConditionedModel
from .dmd_adversarial import Adversary
from .dmd_rollout import Rollout, StudentRollout
from .dmd_schedule import RCM_ENDPOINTS, GANConfig, PhaseClock, Regularization
from .exact_regularization import check_exact_regularization
from .flow import UniformShift, invariant_randn, rf_interpolate, rf_x0, sampling_seeds

__all__ = ["RCM_ENDPOINTS", "DMDModel", "GANConfig", "PhaseClock", "Regularization"]


def _checked_endpoints(values: Sequence[float]) -> tuple[float, ...]:
    levels = tuple(float(v) for v in values)
    descending = all(a > b for a, b in itertools.pairwise(levels))
    if not levels or not descending or not all(0 < v <= 1 for v in levels):
        raise ValueError(f"rollout endpoints must be strictly descending in (0, 1]: {levels}")
    return levels


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
        if (discriminator is None) is not (gan is None):
            raise ValueError("pass both discriminator and gan, or neither")
        levels = _checked_endpoints(rollout_endpoints)
        if block_frames < 1 or int(block_frames) != block_frames:
            raise ValueError(f"block_frames must be a positive integer, got {block_frames}")
        super().__init__(conditioner=conditioner, sampling=sampling,
                         sampling_defaults={"num_steps": len(levels), "seed": 0})
        self.student, self.real_score, self.fake_score = student, real_score, fake_score
        self.discriminator, self.gan = discriminator, gan
        self.block_frames = int(block_frames)
        self.rollout_endpoints = levels
        self.score_time = UniformShift(score_shift)
        self.real_score_guidance = float(real_score_guidance)
        self.clock = PhaseClock(fake_score_updates_per_student, 0 if gan is None else gan.warmup_updates)
        self.dmd_loss_scale = float(dmd_loss_scale)
        self.history = history if history is not None else HistoryWindow()
        self.seed = int(seed)

        unsharded = ParallelConfig(fully_shard=False, compile=False)
        self.student_parallel = student_parallel or unsharded
        self.score_parallel = score_parallel or unsharded
        self.real_score_parallel = real_score_parallel or self.score_parallel
        self.discriminator_parallel = discriminator_parallel or unsharded
        self.conditioner_parallel = conditioner_parallel or self.score_parallel

        self.real_score.requires_grad_(False)
        self.configure_trainable_parameters(student_trainable_patterns, module=self.student)
        self.configure_trainable_parameters(fake_score_trainable_patterns, module=self.fake_score)
        if gan is not None and gan.regularization is Regularization.EXACT:
            if self.real_score_parallel.context_parallel_size > 1:
                raise ValueError("exact R1/R2 does not support context parallelism: its "
                                 "forward-mode pass cannot cross the CP exchange. Use "
                                 "context_parallel_size=1 or finite_difference regularization")
            check_exact_regularization(self.real_score, discriminator)

    # plain (non-module) helpers built on demand: they hold references to registered modules
    @property
    def _rollouts(self) -> StudentRollout:
        return StudentRollout(self.student, self.rollout_endpoints, self.block_frames, self.history)

    @property
    def _adversary(self) -> Adversary:
        if self.gan is None or self.discriminator is None:
            raise RuntimeError("this objective was built without a discriminator")
        return Adversary(self.gan, self.discriminator, self._teacher_features)

    # ------------------------------------------------------------------- lifecycle
    def parallelize(self, device) -> None:
        # the student replays right after a long rollout: keep its parameters gathered
        resident = replace(self.student_parallel, reshard_after_forward=False)
        meshes = [parallelize_network(self.student, resident, device),
                  parallelize_network(self.real_score, self.real_score_parallel, device),
                  parallelize_network(self.fake_score, self.score_parallel, device)]
        self.parallelize_conditioner(self.conditioner_parallel, device)
        if self.discriminator is not None:
            self.discriminator.parallelize(self.discriminator_parallel, device)
        self.real_score.eval()
        self.register_context_parallel_mesh(*meshes)

    def train(self, mode: bool = True) -> "DMDModel":
        super().train(mode)
        self.real_score.eval()  # the teacher never leaves evaluation mode
        return self

    def is_cadence_due(self, iteration: int, interval: int | None) -> bool:
        return self.clock.is_cadence_due(int(iteration), interval)

    def get_optimizer_names(self, iteration: int) -> tuple[str, ...]:
        if self.clock.is_warmup(iteration):
            return ("discriminator",)
        if self.clock.is_student(iteration):
            return ("student",)
        return ("fake_score",) if self.gan is None else ("fake_score", "discriminator")

    def init_optimizer_scheduler(self, optimizer_config, scheduler_config):
        trained = {"student": self.student, "fake_score": self.fake_score}
        if self.discriminator is not None:
            trained["discriminator"] = self.discriminator
        absent = sorted(set(trained) - set(optimizer_config))
        if absent:
            raise KeyError(f"optimizer config lacks roles {absent}")
        self.optimizer_dict = {
            role: instantiate(optimizer_config[role], params=self._group_module_trainable_parameters(module))
            for role, module in trained.items()}
        self.scheduler_dict = {role: instantiate(scheduler_config, optimizer=optimizer)
                               for role, optimizer in self.optimizer_dict.items()}
        return self.optimizer_dict, self.scheduler_dict

    # --------------------------------------------------------------------- rollout
    def _exit_step(self, iteration: int) -> int:
        """The same draw on every rank: a CPU generator seeded from (seed, iteration)."""
        draw = torch.Generator().manual_seed(self.seed * 1_000_003 + iteration)
        return int(torch.randint(len(self.rollout_endpoints), (1,), generator=draw))

    def _validate_rollout(self, frames: int, steps: int) -> None:
        self._rollouts.check(frames, steps)

    def _rollout(self, anchor: Tensor, condition, frames: int, steps: int, *,
                 noise: Tensor | None = None) -> Rollout:
        return self._rollouts.run(anchor, condition, frames, steps, noise=noise)

    # ---------------------------------------------------------------------- scores
    @staticmethod
    def _velocity(network: nn.Module, anchor: Tensor, noisy: Tensor, sigma: Tensor, condition) -> Tensor:
        """A bidirectional score network on [anchor | noisy]: velocity of the noisy frames."""
        clip = torch.cat((anchor, noisy), dim=2)
        return network(clip, sigma, condition, known_frames=1)[:, :, 1:].float()

    def _teacher_features(self, anchor: Tensor, noisy: Tensor, sigma: Tensor, condition):
        """Hidden states of the frozen teacher at the discriminator's layers."""
        clip = torch.cat((anchor, noisy), dim=2)
        return self.real_score(clip, sigma, condition, known_frames=1,
                               feature_layers=self.discriminator.feature_layers)[1]

    def _teacher_velocity(self, anchor, noisy, sigma, prompts) -> Tensor:
        towards = self._velocity(self.real_score, anchor, noisy, sigma, prompts[0])
        if len(prompts) == 1:
            return towards
        away = self._velocity(self.real_score, anchor, noisy, sigma, prompts[1])
        return away + self.real_score_guidance * (towards - away)

    # -------------------------------------------------------------------- closures
    def training_step_closures(self, data_batch: dict[str, Any], iteration: int,
                               ) -> Iterator[TrainingClosureSpec]:
        clip = data_batch["latent"].float()
        anchor, real = clip[:, :, :1], clip[:, :, 1:]
        prompt = self.conditioner.condition(data_batch)
        rollout = self._rollout(anchor, prompt, real.shape[2], self._exit_step(iteration) + 1)
        if self.clock.is_student(iteration):
            prompts = [prompt]
            if self.real_score_guidance != 1.0:
                prompts.append(self.conditioner.condition(data_batch, negative=True))
            yield "student", lambda: self._student_loss(anchor, real, rollout, prompts), True
            return
        idle = self.clock.is_warmup(iteration)
        yield "fake_score", lambda: self._fake_score_loss(anchor, real, rollout.clean, prompt, warmup=idle), True

    def training_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        merged: dict[str, Any] = {}
        total = None
        for _role, closure, _last in self.training_step_closures(data_batch, iteration):
            report, loss = closure()
            merged.update(report)
            total = loss if total is None else total + loss
        return merged, torch.stack([total]).sum()

    def _student_loss(self, anchor, real, rollout: Rollout, prompts) -> StepOutput:
        replayed = self.student.forward_ar(anchor, rollout.noisy, rollout.sigma, prompts[0],
                                           block_frames=self.block_frames, clean=rollout.clean,
                                           history=self.history).float()
        estimate = rf_x0(rollout.noisy, rollout.sigma, replayed)
        target, push, report = self._student_targets(anchor, real, estimate.detach(), prompts)
        matching = self.dmd_loss_scale * (estimate.double() - target.double()).square().sum() / estimate.numel()
        loss = matching.float()
        if push is not None:
            loss = loss + (estimate * push).sum()  # d(loss)/d(estimate) = the GAN gradient
        with torch.no_grad():
            drift = (estimate - rollout.clean).abs().max()
        report["metrics/student/dmd_loss"] = matching.detach()
        report["metrics/student/sgf_recovery_max_abs"] = drift
        report["metrics/student/exit_sigma"] = rollout.sigma[0, 0]
        return report, loss

    def _student_targets(self, anchor, real, estimate, prompts):
        """Detached FP64 target whose squared distance to the estimate has the distribution-
        matching gradient; the GAN gradient (or None); metrics."""
        sigma = self.score_time.sample(estimate.shape[0], device=estimate.device)
        noise = torch.randn_like(estimate)
        with torch.no_grad():
            noisy = rf_interpolate(estimate, noise, sigma)
            by_fake = rf_x0(noisy, sigma, self._velocity(self.fake_score, anchor, noisy, sigma, prompts[0]))
            by_teacher = rf_x0(noisy, sigma, self._teacher_velocity(anchor, noisy, sigma, prompts))
            target, step_rms = ops.dmd_target(estimate, by_fake, by_teacher)
        push, report = None, {}
        if self.gan is not None:
            push, report = self._adversary.generator_gradient(anchor, real, estimate, noise, sigma, prompts[0])
        report["metrics/student/dmd_gradient_rms"] = step_rms
        return target, push, report

    def _fake_score_loss(self, anchor, real, generated, prompt, *, warmup: bool) -> StepOutput:
        sigma = self.score_time.sample(generated.shape[0], device=generated.device)
        noise = torch.randn_like(generated)
        noisy = rf_interpolate(generated, noise, sigma)
        with torch.set_grad_enabled(torch.is_grad_enabled() and not warmup):
            predicted = self._velocity(self.fake_score, anchor, noisy, sigma, prompt)
        regression = (predicted - (noise - generated)).square().mean()
        report = {"metrics/fake_score/loss": regression.detach()}
        loss = regression.detach() * 0 if warmup else regression
        if self.gan is not None:
            judged, judged_report = self._adversary.discriminator_loss(anchor, real, noisy, noise, sigma, prompt)
            loss = loss + judged
            report.update(judged_report)
        return report, loss

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def validation_step(self, data_batch: dict[str, Any], iteration: int) -> StepOutput:
        clip = data_batch["latent"].float()
        anchor, real = clip[:, :, :1], clip[:, :, 1:]
        prompt = self.conditioner.condition(data_batch)
        with isolated_rng():  # a fixed seed per validation batch; the caller's streams stay put
            torch.manual_seed(self.seed)
            rollout = self._rollout(anchor, prompt, real.shape[2], len(self.rollout_endpoints))
            return self._fake_score_loss(anchor, real, rollout.clean, prompt, warmup=False)

    @torch.inference_mode()
    def sample(self, data_batch: dict[str, Any], **options: Any) -> dict[str, Tensor]:
        chosen = self.sampling_options(options)
        clip = data_batch["latent"].float()
        anchor, future = clip[:, :, :1], clip[:, :, 1:]
        self._validate_rollout(future.shape[2], chosen["num_steps"])
        steps = int(chosen["num_steps"])
        seeds = sampling_seeds(data_batch, int(chosen["seed"]))
        prepared = torch.stack([invariant_randn(future, seeds, stream=step) for step in range(steps)])
        rollout = self._rollout(anchor, self.conditioner.condition(data_batch), future.shape[2], steps,
                                noise=prepared)
        panels = dict(self.conditioner.visuals(data_batch))
        panels["ground_truth"] = self.conditioner.decode(clip)
        panels["sample"] = self.conditioner.decode(torch.cat((anchor, rollout.clean), dim=2))
        return panels
