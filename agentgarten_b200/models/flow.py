"""Rectified-flow schedules, batching-invariant noise and the UniPC sampler.

Convention: ``x_sigma = (1 - sigma) * x0 + sigma * noise``; the network predicts the
velocity ``noise - x0``; hence ``x0 = x_sigma - sigma * v``.

Parity: reference ``wm/models/flow.py:33-266``.
"""

from __future__ import annotations

import math
from collections.abc import Callable, Mapping, Sequence
from enum import StrEnum
from typing import Any

import numpy as np
import torch

from agentgarten_b200 import ops

__all__ = [
    "FlowUniPC",
    "RectifiedFlowSchedule",
    "TrainDistribution",
    "UniformShift",
    "VelocityFunction",
    "invariant_randn",
    "rf_interpolate",
    "rf_x0",
    "sampling_seeds",
    "shift_sigma",
]

VelocityFunction = Callable[[torch.Tensor, float], torch.Tensor]


class TrainDistribution(StrEnum):
    UNIFORM = "uniform"
    LOGITNORMAL = "logitnormal"
    WAVER = "waver"


def shift_sigma(sigma: torch.Tensor, shift: float) -> torch.Tensor:
    """Time shift ``s·σ / (1 + (s-1)·σ)`` that moves mass towards high noise for ``s > 1``."""
    return shift * sigma / (1.0 + (shift - 1.0) * sigma)


def rf_interpolate(x0: torch.Tensor, noise: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
    return ops.rf_interpolate(x0, noise, sigma)


def rf_x0(noisy: torch.Tensor, sigma: torch.Tensor, velocity: torch.Tensor) -> torch.Tensor:
    return ops.rf_x0(noisy, sigma, velocity)


def _check_shift(shift: float) -> float:
    if not math.isfinite(shift) or shift <= 0:
        raise ValueError(f"shift must be positive, got {shift}")
    return float(shift)


class RectifiedFlowSchedule:
    """Training-time sigma sampler: uniform, logit-normal or the "waver" mode density."""

    _WAVER_MODE_S = 1.29

    def __init__(self, *, shift: float = 1.0,
                 train_distribution: TrainDistribution | str = TrainDistribution.UNIFORM) -> None:
        self.shift = _check_shift(shift)
        self.train_distribution = TrainDistribution(train_distribution)

    def sample(self, shape: int | Sequence[int], *, device: torch.device,
               generator: torch.Generator | None = None) -> torch.Tensor:
        u = torch.rand(shape, device=device, generator=generator)
        kind = self.train_distribution
        if kind is TrainDistribution.UNIFORM:
            data_time = u
        elif kind is TrainDistribution.LOGITNORMAL:
            data_time = torch.sigmoid(torch.randn(shape, device=device, generator=generator))
        else:
            bump = torch.cos(torch.pi * 0.5 * u).square() - 1.0 + u
            data_time = 1.0 - u - self._WAVER_MODE_S * bump
        return shift_sigma(1.0 - data_time, self.shift)


class UniformShift:
    def __init__(self, shift: float = 5.0) -> None:
        self.shift = _check_shift(shift)

    def sample(self, shape: int | Sequence[int], *, device: torch.device,
               generator: torch.Generator | None = None) -> torch.Tensor:
        return shift_sigma(torch.rand(shape, device=device, generator=generator), self.shift)


def invariant_randn(reference: torch.Tensor, seeds: Sequence[int],
                    dtype: torch.dtype = torch.float32, *, stream: int = 0) -> torch.Tensor:
    """Gaussian noise per sample that depends only on ``(seed, stream)``, never on how
    samples are batched.  Stream 0 is the plain seeded NumPy stream."""
    if len(seeds) != reference.shape[0]:
        raise ValueError(f"need {reference.shape[0]} seeds, got {len(seeds)}")
    shape = tuple(reference.shape[1:])
    draws = []
    for seed in seeds:
        key = int(seed) if stream == 0 else (int(seed), int(stream))
        draws.append(np.random.RandomState(key).standard_normal(shape))
    stacked = np.stack(draws).astype(np.float32)
    return torch.from_numpy(stacked).to(device=reference.device, dtype=dtype)


def sampling_seeds(batch: Mapping[str, Any], seed: int) -> list[int]:
    """``seed + sample_id`` per sample, or ``seed + batch index`` without ids."""
    size = int(batch["latent"].shape[0])
    ids = batch.get("sample_id")
    if ids is None:
        return [seed + i for i in range(size)]
    return [seed + int(v) for v in torch.as_tensor(ids).reshape(-1).tolist()]


class FlowUniPC:
    """Order-2 UniPC (predictor + corrector, ``B(h) = expm1(h)``) on the flow ODE.

    Works on x0-predictions with ``alpha = 1 - sigma`` and half-log-SNR
    ``lambda = log(alpha) - log(sigma)``.  Network timesteps are the integer-truncated
    ``sigma * num_train_timesteps`` (the released solver truncates on purpose).
    """

    order = 2

    def __init__(self, num_steps: int, *, shift: float, num_train_timesteps: int = 1000) -> None:
        top = float(np.float32(1.0 - 1.0 / num_train_timesteps))
        grid = np.linspace(top, 0.0, int(num_steps) + 1)[:-1]
        grid = shift * grid / (1.0 + (shift - 1.0) * grid)
        self.num_train_timesteps = int(num_train_timesteps)
        self.sigmas = torch.from_numpy(np.append(grid, 0.0).astype(np.float32))
        self.timesteps = torch.from_numpy(grid * num_train_timesteps).to(torch.int64)

    def network_sigmas(self) -> torch.Tensor:
        return self.timesteps.float() / self.num_train_timesteps

    @staticmethod
    def _lam(sigma: torch.Tensor) -> torch.Tensor:
        return torch.log(1.0 - sigma) - torch.log(sigma)

    def run(self, sample: torch.Tensor, velocity: VelocityFunction,
            post_step: Callable[[torch.Tensor], torch.Tensor] | None = None) -> torch.Tensor:
        sig = self.sigmas.to(sample.device)
        net_sig = self.network_sigmas()
        total = len(self.timesteps)
        history: list[torch.Tensor] = []  # x0 predictions of earlier steps, oldest first
        previous: torch.Tensor | None = None
        warm = 0          # how many earlier predictions may be used
        used_order = 1    # order of the predictor that produced `sample`
        for i in range(total):
            x0 = sample - sig[i] * velocity(sample, float(net_sig[i])).to(sample.dtype)
            if previous is not None:
                sample = self._correct(x0, history, previous, sig, i, used_order)
            history = [*history[-(self.order - 1):], x0]
            used_order = min(self.order, total - i, warm + 1)
            previous = sample
            sample = self._predict(sample, history, sig, i, used_order)
            warm = min(self.order, warm + 1)
            if post_step is not None:
                sample = post_step(sample)
        return sample

    def _predict(self, x, history, sig, i, order):
        """UniP: from sigma_i to sigma_{i+1}."""
        newest = history[-1]
        s_next, s_now = sig[i + 1], sig[i]
        h = self._lam(s_next) - self._lam(s_now)
        phi = torch.expm1(-h)
        alpha_next = 1.0 - s_next
        out = s_next / s_now * x - alpha_next * phi * newest
        if order == 2:
            r = (self._lam(sig[i - 1]) - self._lam(s_now)) / h
            slope = (history[-2] - newest) / r
            out = out - alpha_next * phi * 0.5 * slope
        return out.to(x.dtype)

    def _correct(self, x0_new, history, x_prev, sig, i, order):
        """UniC: redo the step sigma_{i-1} → sigma_i using the prediction made at sigma_i."""
        base_pred = history[-1]
        s_now, s_prev = sig[i], sig[i - 1]
        h = self._lam(s_now) - self._lam(s_prev)
        hh = -h
        phi1 = torch.expm1(hh)
        big_b = phi1
        phi_k = phi1 / hh - 1.0
        slopes, ratios = [], []
        if order == 2:
            r = (self._lam(sig[i - 2]) - self._lam(s_prev)) / h
            ratios.append(r)
            slopes.append((history[-2] - base_pred) / r)
        ratios.append(1.0)
        device = x_prev.device
        if order == 1:
            rho = torch.tensor([0.5], dtype=x_prev.dtype, device=device)
        else:
            r_vec = torch.tensor([float(v) for v in ratios], device=device)
            rows, rhs, fact = [], [], 1
            for k in range(1, order + 1):
                rows.append(r_vec ** (k - 1))
                rhs.append(phi_k * fact / big_b)
                fact *= k + 1
                phi_k = phi_k / hh - 1.0 / fact
            rho = torch.linalg.solve(
                torch.stack(rows), torch.tensor(rhs, device=device)).to(x_prev.dtype)
        alpha_now = 1.0 - s_now
        out = s_now / s_prev * x_prev - alpha_now * phi1 * base_pred
        past = rho[0] * slopes[0] if slopes else 0
        out = out - alpha_now * big_b * (past + rho[-1] * (x0_new - base_pred))
        return out.to(x_prev.dtype)
