"""The GAN term of Adversarial Forcing: a discriminator head on hidden features of the frozen
teacher, judging noised clips.

``Adversary`` bundles the head, its configuration and the feature extractor, and offers the two
sides of the game:

* ``generator_gradient`` — the gradient of the generator loss with respect to the student's
  clean estimate, obtained with the head frozen (the student receives it as a linear term);
* ``discriminator_loss`` — the (relativistic) pair loss plus the R1/R2 regulariser, either as
  finite differences under small Gaussian jitter or exactly (see
  :mod:`agentgarten_b200.models.exact_regularization`).

Parity: reference ``wm/models/dmd.py:487-620``.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from agentgarten_b200.utils.misc import frozen_parameters

from .dmd_schedule import GANConfig, Regularization
from .exact_regularization import exact_penalties
from .flow import rf_interpolate

__all__ = ["Adversary"]

# (anchor, noisy frames, sigma, condition) -> hidden states at the head's layers
Features = Callable[[Tensor, Tensor, Tensor, Any], tuple[Tensor, ...]]


def _judgement(real: Tensor, fake: Tensor, relativistic: bool) -> Tensor:
    """Discriminator pair loss: ``softplus(fake - real)`` when relativistic, else the sum of the
    two one-sided terms."""
    if relativistic:
        return F.softplus(fake - real).mean()
    return (F.softplus(-real) + F.softplus(fake)).mean()


class Adversary:
    def __init__(self, config: GANConfig, head: nn.Module, features: Features) -> None:
        self.config, self.head, self.features = config, head, features

    # ------------------------------------------------------------------ generator side
    def generator_gradient(self, anchor: Tensor, real: Tensor, estimate: Tensor, noise: Tensor,
                           sigma: Tensor, condition) -> tuple[Tensor, dict[str, Tensor]]:
        config = self.config
        probe = estimate.detach().requires_grad_(True)
        # frozen for the forward, the backward and any recomputation inside this block
        with torch.enable_grad(), frozen_parameters(self.head):
            fake = self.head([self.features(anchor, rf_interpolate(probe, noise, sigma), sigma, condition)])
            with torch.no_grad():
                real_logits = self.head([self.features(anchor, rf_interpolate(real, noise, sigma),
                                                       sigma, condition)])
            margin = fake - real_logits if config.relativistic else fake
            loss = config.generator_weight * F.softplus(-margin).mean()
            (gradient,) = torch.autograd.grad(loss, probe)
        report = {"metrics/student/gan_loss": loss.detach(),
                  "metrics/student/gan_fake_minus_real_logit": margin.detach().mean()}
        return torch.nan_to_num(gradient.detach()), report

    # -------------------------------------------------------------- discriminator side
    def _report(self, pair: Tensor, real: Tensor, fake: Tensor, r1: Tensor | None = None,
                r2: Tensor | None = None) -> dict[str, Tensor]:
        report = {"metrics/discriminator/pair_loss": pair.detach(),
                  "metrics/discriminator/accuracy": (real > fake).float().mean().detach()}
        if r1 is not None:
            report["metrics/discriminator/r1"] = r1.detach()
            report["metrics/discriminator/r2"] = r2.detach()
        return report

    def discriminator_loss(self, anchor: Tensor, real: Tensor, fake_noisy: Tensor, noise: Tensor,
                           sigma: Tensor, condition) -> tuple[Tensor, dict[str, Tensor]]:
        real_noisy = rf_interpolate(real, noise, sigma)
        if self.config.regularization is Regularization.EXACT:
            return self._exact(anchor, real_noisy, fake_noisy, sigma, condition)
        return self._finite_difference(anchor, real_noisy, fake_noisy, sigma, condition)

    def _finite_difference(self, anchor, real_noisy, fake_noisy, sigma, condition):
        config = self.config
        regularised = config.regularization_weight > 0
        stack = [fake_noisy, real_noisy]
        if regularised:
            spread = config.regularization_sigma
            stack.append(real_noisy + spread * torch.randn_like(real_noisy))
            stack.append(fake_noisy + spread * torch.randn_like(fake_noisy))
        copies = len(stack)
        with torch.no_grad():  # one teacher pass over all variants
            hidden = self.features(torch.cat([anchor] * copies), torch.cat(stack), sigma.repeat(copies),
                                   condition.repeat(copies))
        scores = self.head([hidden]).split(fake_noisy.shape[0])
        fake, real = scores[0], scores[1]
        pair = _judgement(real, fake, config.relativistic)
        total = config.discriminator_weight * pair
        if not regularised:
            return total, self._report(pair, real, fake)
        r1 = (scores[2] - real).square().mean()
        r2 = (scores[3] - fake).square().mean()
        total = total + config.discriminator_weight * 0.5 * config.regularization_weight * (r1 + r2)
        return total, self._report(pair, real, fake, r1, r2)

    def _exact(self, anchor, real_noisy, fake_noisy, sigma, condition):
        config = self.config
        count = fake_noisy.shape[0]
        both_anchor, both_sigma, both_condition = torch.cat((anchor, anchor)), sigma.repeat(2), condition.repeat(2)

        def hidden(rows: Tensor) -> tuple[Tensor, ...]:
            return self.features(both_anchor, rows, both_sigma, both_condition)

        outcome = exact_penalties(hidden, self.head, torch.cat((fake_noisy, real_noisy)))
        fake, real = outcome.logits.split(count)
        r2, r1 = (part.mean() for part in outcome.penalty.split(count))
        pair = _judgement(real, fake, config.relativistic)
        # value: the weighted penalties; gradient: carried by the zero-valued surrogate
        carried = outcome.surrogate.view(2, count).mean(1).sum()
        weight = config.discriminator_weight * 0.5 * config.exact_regularization_weight
        total = config.discriminator_weight * pair + weight * ((r1 + r2) + carried)
        return total, self._report(pair, real, fake, r1, r2)
