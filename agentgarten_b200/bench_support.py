"""Construction of the flagship training job from synthetic data and random weights.

Used by ``bench.py`` and the smoke check: builds the bidirectional rectified-flow objective
(generation tower + frozen text tower) at a requested size, initialises weights randomly on
the device and returns an object whose ``step(batch)`` runs one complete update through the
public training API: ``prepare_data_batch`` → ``training_step`` → ``backward`` → gradient
clipping → ``FusedAdam.step`` → ``zero_grad``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from agentgarten_b200.infra.optim import FusedAdam
from agentgarten_b200.models.diffusion import DiffusionModel
from agentgarten_b200.models.flow import RectifiedFlowSchedule
from agentgarten_b200.networks.cosmos3 import Cosmos3Config, build_network
from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
from agentgarten_b200.parallel import zero
from agentgarten_b200.parallel.engine import ParallelConfig

__all__ = ["TrainingJob", "build_training_job", "random_init_", "synthetic_batch"]


@torch.no_grad()
def random_init_(module: torch.nn.Module, seed: int = 0, std: float = 0.02) -> None:
    """Random weights of the architecture: N(0, std) matrices and embeddings, unit norms,
    zero biases.  Generated on the parameter's device, one parameter at a time."""
    generator = torch.Generator(device=next(module.parameters()).device)
    generator.manual_seed(seed)
    for name, p in module.named_parameters():
        if p.ndim >= 2:
            p.normal_(0.0, std, generator=generator)
        elif "norm" in name:
            p.fill_(1.0)
        elif name.endswith("bias"):
            p.zero_()
        else:
            p.normal_(0.0, std, generator=generator)


@dataclass
class TrainingJob:
    model: DiffusionModel
    optimizer: FusedAdam
    config: Cosmos3Config
    device: torch.device
    frames: int
    latent_hw: tuple[int, int]
    text_tokens: int
    max_grad_norm: float = 1.0
    grad_accum_steps: int = 1
    extras: dict[str, Any] = field(default_factory=dict)

    @property
    def rgb_tokens_per_clip(self) -> int:
        p = self.config.patch_size
        return self.frames * (self.latent_hw[0] // p) * (self.latent_hw[1] // p)

    def step(self, batch: dict[str, Any], stage: Any = None) -> torch.Tensor:
        """One optimizer update; returns the (device) loss of the last microbatch.  ``stage``
        (optional) maps the batch to the device copy of one microbatch, so that every
        microbatch of an end-to-end measurement makes its own host-to-device transfer."""
        model, optimizer = self.model, self.optimizer
        loss = None
        for micro in range(self.grad_accum_steps):
            zero.arm_overlap(micro == self.grad_accum_steps - 1)
            encoded = model.prepare_data_batch(batch if stage is None else stage(batch))
            _, loss = model.training_step(encoded, 0)
            (loss / self.grad_accum_steps).backward()
        norm_sq = optimizer.grad_norm_sq()
        # clip coefficient stays on the device: min(1, max_norm / (norm + 1e-6))
        coef = (self.max_grad_norm / (norm_sq.sqrt() + 1e-6)).clamp(max=1.0)
        optimizer.grad_scale = coef
        optimizer.step()
        optimizer.zero_grad()
        return loss.detach()


def build_training_job(device: torch.device | str, *, layers: int = 36, hidden: int = 4096,
                       intermediate: int = 12288, heads: int = 32, kv_heads: int = 8,
                       vocab: int = 151936, frames: int = 21, latent_hw: tuple[int, int] = (30, 52),
                       text_tokens: int = 512, text_layers: int | None = None, lr: float = 3e-5,
                       seed: int = 0, fully_shard: bool = True,
                       recipe: str = "bidirectional", context_parallel: int = 1) -> TrainingJob:
    """``recipe``: ``bidirectional`` (rectified flow on the whole clip), ``ar_diffusion_forcing``
    or ``ar_teacher_forcing`` (block-causal, blocks of 4 latent frames after the anchor).
    ``context_parallel`` ranks share one clip (Ulysses sharding of the generation tower)."""
    device = torch.device(device)
    config = Cosmos3Config(hidden_size=hidden, intermediate_size=intermediate,
                           num_hidden_layers=layers, num_attention_heads=heads,
                           num_key_value_heads=kv_heads, vocab_size=vocab)
    text_config = config if text_layers is None else Cosmos3Config(
        hidden_size=hidden, intermediate_size=intermediate, num_hidden_layers=text_layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, vocab_size=vocab)
    net = build_network(config, init_device="meta")
    conditioner = Cosmos3Conditioner(config=text_config, codec=None, init_device="meta",
                                     geometry_noise_sigma=0.0)
    parallel = ParallelConfig(parameter_dtype="bfloat16", fully_shard=fully_shard,
                              context_parallel_size=context_parallel,
                              activation_checkpointing="selective", compile=False)
    frozen = ParallelConfig(parameter_dtype="bfloat16", fully_shard=fully_shard,
                            activation_checkpointing="none", compile=False)
    schedule = RectifiedFlowSchedule(shift=5.0, train_distribution="waver")
    if recipe == "bidirectional":
        model = DiffusionModel(net=net, conditioner=conditioner, schedule=schedule,
                               text_dropout=0.1, parallel=parallel, conditioner_parallel=frozen)
    elif recipe in ("ar_diffusion_forcing", "ar_teacher_forcing"):
        from agentgarten_b200.models.autoregressive import AutoregressiveModel

        model = AutoregressiveModel(net=net, conditioner=conditioner, schedule=schedule,
                                    mode=recipe.removeprefix("ar_"), block_frames=4, text_dropout=0.1,
                                    parallel=parallel, conditioner_parallel=frozen)
    else:
        raise ValueError(f"unknown recipe {recipe!r}")
    model.parallelize(device)
    random_init_(model.net, seed=seed)
    random_init_(model.conditioner.text_encoder, seed=seed + 1)
    model.train()
    optimizer = FusedAdam(model._group_trainable_parameters(), lr=lr, betas=(0.9, 0.99), eps=1e-8,
                          weight_decay=0.0, adam_w_mode=True, use_te_capturable_kernel=True,
                          master_weights=True)
    return TrainingJob(model=model, optimizer=optimizer, config=config, device=device,
                       frames=frames, latent_hw=latent_hw, text_tokens=text_tokens)


def synthetic_batch(job: TrainingJob, device: torch.device | str = "cpu", seed: int = 0,
                    pinned: bool = False) -> dict[str, Any]:
    """Cached-latent batch of one clip: latent / depth / normal ``[1, 48, T, H, W]`` ~ N(0,1),
    prompt ids ``[1, text_tokens]``; the VAE and the tokenizer are bypassed."""
    g = torch.Generator().manual_seed(seed)
    c = job.config.latent_channels
    shape = (1, c, job.frames, *job.latent_hw)
    batch = {
        "latent": torch.randn(shape, generator=g),
        "depth_latent": torch.randn(shape, generator=g),
        "normal_latent": torch.randn(shape, generator=g),
        "text_input_ids": torch.randint(1000, min(job.config.vocab_size, 150000),
                                        (1, job.text_tokens), generator=g),
        "fps": torch.full((1,), 16.0),
    }
    if pinned:
        batch = {k: v.pin_memory() for k, v in batch.items()}
    if torch.device(device).type != "cpu":
        batch = {k: v.to(device, non_blocking=True) for k, v in batch.items()}
    return batch


def batch_bytes(batch: dict[str, Any]) -> int:
    return sum(v.numel() * v.element_size() for v in batch.values() if isinstance(v, torch.Tensor))
