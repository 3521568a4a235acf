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

__all__ = ["TrainingJob", "build_training_job", "random_init_", "stream_benchmark", "synthetic_batch"]


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


def stream_benchmark(device: torch.device, *, blocks: int = 32, layers: int = 36, graphs: bool = True,
                     tensor_parallel: bool = False, trace: bool = False) -> dict[str, Any]:
    """Cosmos3Stream on synthetic inputs: batch 1, anchor ``[1, 48, 1, 30, 52]``, ``blocks`` blocks
    of 4 latent frames, each 4 denoise steps at sigma (1.0, 0.75, 0.5, 0.25) and a commit into a
    cache of 6 blocks plus the anchor.  With an initialised process group of more than one rank
    (or ``tensor_parallel``) the tower is sharded over the ranks, which must all call this with
    the same arguments.  Every cache fill level's CUDA graph is captured before the first timed
    block; ALL blocks count.  Returns per-block device times (max over ranks) and their
    p50 / p99."""
    import statistics

    import torch.distributed as dist

    from agentgarten_b200.inference.serving import prepare_serving, release_serving
    from agentgarten_b200.models.flow import rf_interpolate, rf_x0
    from agentgarten_b200.networks.cosmos3.network import Cosmos3Condition
    from agentgarten_b200.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy
    from agentgarten_b200.ops import native

    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    config = Cosmos3Config(num_hidden_layers=layers)
    net = build_network(config, init_device="meta").to(torch.bfloat16).to_empty(device=device)
    random_init_(net, seed=0)
    cond = Cosmos3Conditioner(config=config, codec=None, init_device="meta", geometry_noise_sigma=0.0)
    cond.to(torch.bfloat16).to_empty(device=device)
    random_init_(cond.text_encoder, seed=1)
    sharded = world > 1 or tensor_parallel
    graphs = graphs and not trace
    prepare_serving(net, cuda_graphs=graphs, tensor_parallel=True if sharded else None, max_tokens=4096)
    policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=24, rope="top_aligned",
                          train_frames=61)
    g = torch.Generator(device=device).manual_seed(0)
    shape = (1, 48, 4, 30, 52)
    ids = torch.randint(1000, 150000, (1, 512), device=device, generator=g)
    with torch.inference_mode():
        text = cond.text_encoder(ids, None)
    del cond

    def condition(frames):
        s = (1, 48, frames, 30, 52)
        return Cosmos3Condition(text=text, depth=torch.randn(s, device=device, generator=g),
                                normal=torch.randn(s, device=device, generator=g),
                                fps=torch.full((1,), 16.0, device=device))

    endpoints = (1.0, 0.75, 0.5, 0.25)
    stream = Cosmos3Stream(net, policy)
    anchor = torch.randn((1, 48, 1, 30, 52), device=device, generator=g)
    stream.capture_graphs(anchor, condition(1), condition(4))   # before the timed blocks
    stream.start(anchor, condition(1))
    times: list[float] = []
    launches_before = native.launches()
    for block in range(blocks):
        if trace and sharded and block == blocks - 2:
            net._tensor_parallel.trace = {}
        cond_block = condition(4)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        clean = None
        for sigma in endpoints:
            level = torch.full((1,), sigma, device=device)
            noise = torch.randn(shape, device=device, generator=g)
            current = noise if clean is None else rf_interpolate(clean, noise, level)
            clean = rf_x0(current, level, stream.denoise(current, level, cond_block))
        stream.commit(clean, cond_block)
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
        # a bounded wait that ran out on any rank ends the run on all of them (outside the timing)
        failed = native.ext().status(device.index).clone()
        if world > 1:
            dist.all_reduce(failed, op=dist.ReduceOp.MAX)
        if int(failed.item()) != 0:
            break
    status = int(native.ext().status(device.index).item())
    if world > 1:
        gathered = torch.tensor(times + [float(status)], device=device)  # same length on every rank
        dist.all_reduce(gathered, op=dist.ReduceOp.MAX)
        times, status = gathered[:-1].tolist(), int(gathered[-1].item())
    phases = net._tensor_parallel.trace_summary() if trace and sharded else None
    launches = native.launches() - launches_before
    release_serving(net)
    ordered = sorted(times)
    return {
        "metric": "Cosmos3Stream ms per 4-frame block (4 denoise + 1 commit)",
        "p50_ms": statistics.median(times),
        "p99_ms": ordered[min(len(ordered) - 1, int(0.99 * len(ordered)))],
        "mean_ms": statistics.fmean(times),
        "first_blocks_ms": times[:8], "blocks": blocks, "n_gpus": world, "dtype": "bf16",
        "parallelism": f"tp{world} (heads and MLP columns; GEMM+reduce-scatter / all-gather+GEMM over peer memory)"
        if sharded else "single GPU",
        "cuda_graphs": graphs, "layers": layers,
        "cache": "anchor + 6 blocks (sink 1, history 24 frames), top-aligned RoPE",
        "tokens_per_block": 4 * 2 * 390, "gpu_launches": launches, "kernel_status": status,
        "timed": "all blocks; every fill-level graph captured beforehand",
        **({"phase_ms": phases} if phases is not None else {}),
    }
