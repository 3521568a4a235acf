"""Adversarial Forcing (DMD + discriminator with exact R1/R2) step time on synthetic data.

``python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench_dmd.py``

Builds the objective of the ``cosmos3/dmd_gan_exact`` recipe at the Cosmos3-Nano shape with
random weights (student, frozen teacher, fake score, discriminator head on teacher features,
frozen text tower), places it with the sharded optimizer engine and drives it through
``Trainer.training_step`` — the call the training loop makes.  One cycle is one student
update followed by ``--fake-score-updates`` fake-score updates (the discriminator is updated
with the fake score); after one untimed cycle, ``--cycles`` cycles are timed with CUDA events
between barriers and the maximum over ranks is reported as seconds per step (mean over the
iterations of a cycle) and per role.

The three 7 B towers carry two FP32 optimizer states: the full size needs the 8 GPUs of a
node.  ``--layers`` shrinks the towers for a functional check on fewer GPUs; a number taken
that way is not the benchmark.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

# The exact R1/R2 pass of a fake-score update runs while that tower's kept activations are
# alive and needs tens of GB for its forward-mode tangents: the layers keep fewer activations
# (they recompute instead) so that the pass has room, and the allocator may grow its segments
# instead of failing on fragmentation.  Both are defaults that the environment can override.
os.environ.setdefault("AGB200_ACTIVATION_RESERVE_GB", "72")
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def parse_args() -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--cycles", type=int, default=2)
    parser.add_argument("--fake-score-updates", type=int, default=5)
    parser.add_argument("--layers", type=int, default=36, help="smaller values are for checking only")
    parser.add_argument("--blocks", type=int, default=3, help="rollout blocks of 4 latent frames")
    parser.add_argument("--regularization", default="exact", choices=["exact", "finite_difference"])
    return parser.parse_args()


def build(device, args):
    import torch

    from agentgarten_b200.bench_support import random_init_
    from agentgarten_b200.infra.config import LazyCall
    from agentgarten_b200.infra.optim import FusedAdam, LinearWarmup
    from agentgarten_b200.models.dmd import DMDModel, GANConfig
    from agentgarten_b200.networks.cosmos3 import Cosmos3Config, build_network
    from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
    from agentgarten_b200.networks.discriminator import DiscriminatorHead
    from agentgarten_b200.parallel.engine import ParallelConfig

    config = Cosmos3Config(num_hidden_layers=args.layers)
    taps = tuple(sorted({args.layers // 3 - 1, 2 * args.layers // 3 - 1, args.layers - 1} - {-1}))

    def tower():
        return build_network(config, init_device="meta")

    def parallel(checkpointing: str, dtype: str = "bfloat16") -> ParallelConfig:
        return ParallelConfig(parameter_dtype=dtype, fully_shard=True,
                              activation_checkpointing=checkpointing, compile=False)

    head = DiscriminatorHead(hidden_size=config.hidden_size, feature_layers=taps, mlp_ratio=4.0,
                             num_heads=config.num_attention_heads, initial_logit_sign=-1.0,
                             init_device="meta")
    gan = GANConfig(generator_weight=0.01, discriminator_weight=0.01, relativistic=True,
                    regularization=args.regularization, exact_regularization_weight=0.075,
                    warmup_updates=0)
    model = DMDModel(
        student=tower(), real_score=tower(), fake_score=tower(),
        conditioner=Cosmos3Conditioner(config=config, codec=None, init_device="meta",
                                       geometry_noise_sigma=0.0),
        discriminator=head, gan=gan, block_frames=4, score_shift=5.0, real_score_guidance=6.0,
        fake_score_updates_per_student=args.fake_score_updates, dmd_loss_scale=0.5,
        student_parallel=parallel("full"), score_parallel=parallel("full"),
        real_score_parallel=parallel("full"), conditioner_parallel=parallel("none"),
        discriminator_parallel=parallel("full", "float32"), sampling={"num_steps": 4, "seed": 2026})
    model.parallelize(device)
    # the discriminator head initialises itself from its own seed when it is placed
    for seed, module in enumerate((model.student, model.real_score, model.fake_score,
                                   model.conditioner.text_encoder)):
        random_init_(module, seed=seed)
    model.train()

    def adam(lr: float):
        return LazyCall(FusedAdam)(lr=lr, betas=(0.0, 0.999), eps=1e-8, weight_decay=0.0,
                                   adam_w_mode=True, use_te_capturable_kernel=True, master_weights=True)

    schedule = LazyCall(torch.optim.lr_scheduler.LambdaLR)(lr_lambda=LazyCall(LinearWarmup)(warmup_steps=1))
    model.init_optimizer_scheduler({"student": adam(2e-6), "fake_score": adam(4e-7),
                                    "discriminator": adam(2e-7)}, schedule)
    return model, config


def main() -> int:
    args = parse_args()
    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from agentgarten_b200.infra import distributed
    from agentgarten_b200.infra.trainer import Trainer
    from agentgarten_b200.ops import native

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    device = distributed.init(device="cuda", backend="nccl")
    rank, world = distributed.get_rank(), int(os.environ.get("WORLD_SIZE", "1"))
    native.require()
    model, config = build(device, args)
    trainer = Trainer(grad_accum_steps=1, callbacks=None, device=device)

    frames = 1 + 4 * args.blocks
    g = torch.Generator().manual_seed(1000 + rank)
    shape = (1, config.latent_channels, frames, 30, 52)
    batch = {"latent": torch.randn(shape, generator=g), "depth_latent": torch.randn(shape, generator=g),
             "normal_latent": torch.randn(shape, generator=g),
             "text_input_ids": torch.randint(1000, 150000, (1, 512), generator=g),
             "fps": torch.full((1,), 16.0)}
    batch = {k: v.pin_memory() for k, v in batch.items()}

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cycle = args.fake_score_updates + 1
    iteration = 0

    def one(i: int) -> None:
        staged = {k: v.to(device, non_blocking=True) for k, v in batch.items()}
        trainer.training_step(model, None, model.prepare_data_batch(staged), iteration=i)

    for _ in range(cycle):  # one untimed cycle: allocations, first-use set-up
        one(iteration)
        iteration += 1
    barrier()
    launches_before = native.launches()
    per_iteration: list[tuple[str, float]] = []
    for _ in range(args.cycles * cycle):
        role = "student" if model.clock.is_student(iteration) else "fake_score"
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        one(iteration)
        stop.record()
        barrier()
        per_iteration.append((role, start.elapsed_time(stop)))
        iteration += 1
    times = torch.tensor([ms for _, ms in per_iteration], device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    times = times.tolist()
    status = int(native.ext().status(device.index or 0).item())
    if rank == 0:
        by_role: dict[str, list[float]] = {}
        for (role, _), ms in zip(per_iteration, times):
            by_role.setdefault(role, []).append(ms)
        print(json.dumps({
            "metric": "Adversarial Forcing s/step (mean over one student + fake-score cycle)",
            "value": sum(times) / len(times) / 1e3, "unit": "s/step", "higher_is_better": False,
            "n_gpus": world, "cycles": args.cycles, "iterations": len(times),
            "s_per_step_by_role": {k: sum(v) / len(v) / 1e3 for k, v in by_role.items()},
            "dtype": "bf16", "data": "synthetic cached latents N(0,1), random-init weights",
            "config": {"model": f"student / teacher / fake score: {config.num_hidden_layers} layers, hidden "
                                f"{config.hidden_size}; discriminator head on teacher features; frozen text tower",
                       "rollout": f"{args.blocks} blocks of 4 latent frames at 30x52, 4 sigma endpoints",
                       "regularization": args.regularization, "global_batch": world,
                       "fake_score_updates_per_student": args.fake_score_updates,
                       "parallelism": f"dp{world}, sharded FP32 optimizer state"},
            "gpu_launches": native.launches() - launches_before, "kernel_status": status,
            "peak_memory_gb": round(torch.cuda.max_memory_allocated(device) / 2 ** 30, 1),
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
