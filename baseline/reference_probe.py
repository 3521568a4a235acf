"""Golden outputs of the UNMODIFIED reference package for the parity tests.

Runs with ``PYTHONPATH=baseline/_ref:baseline/shims`` (nothing of ``agentgarten_b200`` is
imported).  ``network`` mode builds a small generation tower and text tower on the CPU in
FP32, runs ``forward``, ``forward_ar`` (diffusion and teacher forcing), a cached rollout
(``prefill`` / ``denoise`` / ``commit``) and a streamed block, and writes the state dicts,
the inputs and every output to one ``torch.save`` file.  ``train`` mode runs seeded
optimizer updates through the reference ``Trainer`` and writes the loss sequence and the
final parameters.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch


def tiny_config():
    from wm.networks.cosmos3 import Cosmos3Config

    return Cosmos3Config(hidden_size=256, intermediate_size=1024, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=128,
                         mrope_section=(12, 10, 10), text_bucket_tokens=16,
                         special_tokens={"eos_token_id": 1, "start_of_generation": 2})


def seeded_(module: torch.nn.Module, seed: int) -> None:
    """Seeded full tensors, the same on every rank; a sharded parameter keeps its own chunk."""
    from torch.distributed.tensor import DTensor, distribute_tensor

    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in module.named_parameters():
            if p.ndim >= 2 or "embed" in name:
                full = torch.randn(p.shape, generator=g) * 0.02
            elif "norm" in name:
                full = 1.0 + 0.1 * torch.randn(p.shape, generator=g)
            else:
                full = torch.randn(p.shape, generator=g) * 0.02
            if isinstance(p, DTensor):
                p.to_local().copy_(distribute_tensor(full, p.device_mesh, p.placements).to_local())
            else:
                p.copy_(full)


def batch_of(frames: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    shape = (1, 48, frames, 8, 8)
    return {"latent": torch.randn(shape, generator=g), "depth_latent": torch.randn(shape, generator=g),
            "normal_latent": torch.randn(shape, generator=g),
            "text_input_ids": torch.randint(3, 128, (1, 10), generator=g), "fps": torch.full((1,), 16.0)}


def network_mode(path: str) -> None:
    from wm.codecs import Wan22VAECodec
    from wm.models.flow import rf_interpolate
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network
    from wm.networks.cosmos3.network import Cosmos3Condition
    from wm.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy

    config = tiny_config()
    net = build_network(config, init_device="cpu").float().eval()
    seeded_(net, 0)
    cond = Cosmos3Conditioner(config=config, codec=Wan22VAECodec(pretrained_path="unused", decoder=None),
                              geometry_noise_sigma=0.0, init_device="cpu", empty_prompt_ids=(3, 4, 5)).float()
    seeded_(cond.text_encoder, 1)
    batch = cond.encode(batch_of(9), training=False)
    condition = cond.condition(batch)
    latent = batch["latent"]
    g = torch.Generator().manual_seed(5)
    noise = torch.randn(latent.shape, generator=g)
    out: dict = {"net": net.state_dict(), "text_encoder": cond.text_encoder.state_dict(),
                 "batch": batch_of(9), "noise": noise}
    with torch.no_grad():
        sigma = torch.tensor([0.7])
        noisy = rf_interpolate(latent, noise, sigma)
        noisy[:, :, :1] = latent[:, :, :1]
        out["forward"] = net(noisy, sigma, condition, known_frames=1)
        block_sigma = torch.tensor([[0.9] * 4 + [0.3] * 4])
        targets = rf_interpolate(latent[:, :, 1:], noise[:, :, 1:], block_sigma)
        out["block_sigma"] = block_sigma
        out["forward_ar"] = net.forward_ar(latent[:, :, :1], targets, block_sigma, condition,
                                           block_frames=4)
        out["forward_ar_teacher"] = net.forward_ar(latent[:, :, :1], targets, block_sigma, condition,
                                                   block_frames=4, clean=latent[:, :, 1:])
        cache = net.prefill(latent[:, :, :1], condition)
        first = net.denoise(cache, targets[:, :, :4], torch.tensor([0.9]))
        cache = net.commit(cache, latent[:, :, 1:5])
        second = net.denoise(cache, targets[:, :, 4:], torch.tensor([0.3]))
        out["cached"] = (first, second)

        def part(lo: int, hi: int) -> Cosmos3Condition:
            return Cosmos3Condition(text=condition.text, depth=condition.depth[:, :, lo:hi],
                                    normal=condition.normal[:, :, lo:hi], fps=condition.fps)

        stream = Cosmos3Stream(net, StreamPolicy(block_frames=4, sink_frames=1, history_frames=4,
                                                 rope="top_aligned", train_frames=9))
        stream.start(latent[:, :, :1], part(0, 1))
        streamed = []
        for block in range(2):
            lo, hi = 1 + 4 * block, 5 + 4 * block
            streamed.append(stream.denoise(targets[:, :, lo - 1:hi - 1], torch.tensor([0.6]), part(lo, hi)))
            stream.commit(latent[:, :, lo:hi], part(lo, hi))
        out["streamed"] = tuple(streamed)
        out["stream_keys"] = [key.clone() for key in stream.keys]
    torch.save(out, path)


def train_mode(path: str, steps: int) -> None:
    from wm.codecs import Wan22VAECodec
    from wm.infra.callbacks import CallbackGroup, GradClip
    from wm.infra.config import LazyCall
    from wm.infra.optim import FusedAdam, LinearWarmup
    from wm.infra.parallel import ParallelConfig
    from wm.infra.trainer import Trainer
    from wm.models.diffusion import DiffusionModel
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network

    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)
    model = DiffusionModel(
        net=build_network(config, init_device="cpu"),
        conditioner=Cosmos3Conditioner(config=config, geometry_noise_sigma=0.0, init_device="cpu",
                                       empty_prompt_ids=(3, 4, 5),
                                       codec=Wan22VAECodec(pretrained_path="unused", decoder=None)),
        text_dropout=0.1, parallel=plain, conditioner_parallel=plain)
    model.parallelize("cpu")
    seeded_(model.net, 0)
    seeded_(model.conditioner.text_encoder, 1)
    model.train()
    optimizer = FusedAdam(model._group_trainable_parameters(), lr=1e-3, betas=(0.9, 0.99), eps=1e-8,
                          weight_decay=0.01, adam_w_mode=True, use_te_capturable_kernel=True,
                          master_weights=True)
    scheduler = torch.optim.lr_scheduler.LambdaLR(
        optimizer, lr_lambda=LinearWarmup(warmup_steps=4, start_factor=0.1))
    model.optimizer_dict, model.scheduler_dict = {"net": optimizer}, {"net": scheduler}
    callbacks = CallbackGroup(
        {"trainer": {"callbacks": {"grad_clip": LazyCall(GradClip)(max_norm=1.0)}}}, trainer=None)
    trainer = Trainer(grad_accum_steps=2, callbacks=callbacks, device=torch.device("cpu"))
    scaler = torch.amp.GradScaler(device="cpu", enabled=False)
    torch.manual_seed(1234)
    losses = []
    for step in range(steps):
        for micro in range(2):
            data = trainer._prepare_data_batch(model, batch_of(5, seed=10 * step + micro))
            result = trainer.training_step(model, scaler, data, iteration=step, grad_accum_step=micro)
            losses.append(float(result.loss))
    torch.save({"losses": losses, "net": model.net.state_dict(),
                "lr": optimizer.param_groups[0]["lr"]}, path)


def autoregressive_mode(path: str) -> None:
    """Training and validation losses of the block-causal objective in both forcing modes
    (teacher forcing with degraded history), and their gradients' norm."""
    from wm.codecs import Wan22VAECodec
    from wm.models.autoregressive import AutoregressiveModel, corrupt_history
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network
    from wm.infra.parallel import ParallelConfig

    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)
    out: dict = {}
    for mode in ("teacher_forcing", "diffusion_forcing"):
        model = AutoregressiveModel(
            net=build_network(config, init_device="cpu"),
            conditioner=Cosmos3Conditioner(config=config, geometry_noise_sigma=0.0, init_device="cpu",
                                           empty_prompt_ids=(3, 4, 5),
                                           codec=Wan22VAECodec(pretrained_path="unused", decoder=None)),
            mode=mode, block_frames=4, text_dropout=0.5, parallel=plain, conditioner_parallel=plain)
        model.parallelize("cpu")
        seeded_(model.net, 0)
        seeded_(model.conditioner.text_encoder, 1)
        model.train()
        data = model.prepare_data_batch(batch_of(9, seed=3))
        torch.manual_seed(77)
        report, loss = model.training_step(data, 0)
        loss.backward()
        norm = torch.sqrt(sum(p.grad.square().sum() for p in model.net.parameters() if p.grad is not None))
        model.eval()
        _, validation = model.validation_step(model.prepare_data_batch(batch_of(9, seed=4)), 0)
        out[mode] = {"loss": float(loss), "sigma": report["sigma"], "grad_norm": float(norm),
                     "validation": float(validation)}
    g = torch.Generator().manual_seed(5)
    frames = torch.randn(2, 6, 7, 12, 10, generator=g)
    out["corrupted"] = corrupt_history(frames, torch.Generator().manual_seed(6))
    out["frames"] = frames
    torch.save(out, path)


def dmd_mode(path: str) -> None:
    """Adversarial Forcing on small towers: the loss and the reported metrics of a discriminator
    warm-up iteration, a student iteration and a fake-score + discriminator iteration, for the
    finite-difference and the exact R1/R2 regularisation; plus a validation step."""
    from wm.codecs import Wan22VAECodec
    from wm.infra.parallel import ParallelConfig
    from wm.models.dmd import DMDModel, GANConfig
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network
    from wm.networks.discriminator import DiscriminatorHead

    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)
    out: dict = {}
    for kind in ("finite_difference", "exact"):
        towers = [build_network(config, init_device="cpu") for _ in range(3)]
        for index, tower in enumerate(towers):
            seeded_(tower, 20 + index)
        head = DiscriminatorHead(hidden_size=256, feature_layers=(0, 1), mlp_ratio=2.0, num_heads=4,
                                 init_device="cpu")
        model = DMDModel(
            student=towers[0], real_score=towers[1], fake_score=towers[2],
            conditioner=Cosmos3Conditioner(config=config, geometry_noise_sigma=0.0, init_device="cpu",
                                           empty_prompt_ids=(3, 4, 5),
                                           codec=Wan22VAECodec(pretrained_path="unused", decoder=None)),
            discriminator=head, gan=GANConfig(regularization=kind, warmup_updates=1),
            block_frames=4, fake_score_updates_per_student=2, student_parallel=plain,
            score_parallel=plain, discriminator_parallel=plain, seed=3)
        model.parallelize("cpu")
        seeded_(model.conditioner.text_encoder, 1)
        model.train()
        record: dict = {"head": {k: v.clone() for k, v in head.state_dict().items()}}
        data = model.prepare_data_batch(batch_of(9, seed=8))
        for iteration in range(3):
            torch.manual_seed(100 + iteration)
            model.zero_grad(set_to_none=True)
            report, loss = model.training_step(data, iteration)
            loss.backward()
            grads = {name: float(sum(float(p.grad.double().square().sum()) for p in module.parameters()
                                     if p.grad is not None)) ** 0.5
                     for name, module in (("student", model.student), ("fake_score", model.fake_score),
                                          ("discriminator", head))}
            record[iteration] = {"loss": float(loss), "grads": grads,
                                 "names": model.get_optimizer_names(iteration),
                                 "report": {k: float(v) for k, v in report.items() if torch.is_tensor(v) and v.numel() == 1}}
        model.eval()
        _, validation = model.validation_step(data, 0)
        record["validation"] = float(validation)
        out[kind] = record
    torch.save(out, path)


def checkpoint_mode(path: str, directory: str, resume: bool) -> None:
    """Two or more Gloo ranks, FSDP2.  Without ``resume``: two updates, a checkpoint
    ``iter_000000002`` under ``directory``, a third update; with it: load ``directory/latest``
    (written by either implementation) into a fresh job and run the third update.  The loss
    of the third update (mean over ranks) is written to ``path`` by rank 0."""
    import torch.distributed as dist

    from wm.codecs import Wan22VAECodec
    from wm.infra import distributed
    from wm.infra.checkpoint import DistributedCheckpointer
    from wm.infra.callbacks import CallbackGroup, GradClip
    from wm.infra.config import LazyCall
    from wm.infra.optim import FusedAdam, LinearWarmup
    from wm.infra.parallel import ParallelConfig
    from wm.infra.trainer import Trainer
    from wm.models.diffusion import DiffusionModel
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network

    device = distributed.init(device="cpu", backend="gloo")
    rank = distributed.get_rank()
    config = tiny_config()
    sharded = ParallelConfig(parameter_dtype="float32", fully_shard=True, activation_checkpointing="none",
                             compile=False)
    model = DiffusionModel(
        net=build_network(config, init_device="meta"),
        conditioner=Cosmos3Conditioner(config=config, geometry_noise_sigma=0.0, init_device="meta",
                                       empty_prompt_ids=(3, 4, 5),
                                       codec=Wan22VAECodec(pretrained_path="unused", decoder=None)),
        text_dropout=0.0, parallel=sharded, conditioner_parallel=sharded)
    model.parallelize(device)
    seeded_(model.net, 0 if not resume else 50)  # a resumed job starts from other weights
    seeded_(model.conditioner.text_encoder, 1)
    model.train()
    optimizer = FusedAdam(model._group_trainable_parameters(), lr=1e-3, betas=(0.9, 0.99), eps=1e-8,
                          weight_decay=0.01, adam_w_mode=True, use_te_capturable_kernel=True,
                          master_weights=True)
    scheduler = torch.optim.lr_scheduler.LambdaLR(
        optimizer, lr_lambda=LinearWarmup(warmup_steps=4, start_factor=0.1))
    model.optimizer_dict, model.scheduler_dict = {"net": optimizer}, {"net": scheduler}
    callbacks = CallbackGroup(
        {"trainer": {"callbacks": {"grad_clip": LazyCall(GradClip)(max_norm=1.0)}}}, trainer=None)
    trainer = Trainer(grad_accum_steps=1, callbacks=callbacks, device=device)
    scaler = torch.amp.GradScaler(device="cpu", enabled=False)
    checkpointer = DistributedCheckpointer(directory, async_mode="disabled")

    def update(step: int) -> float:
        torch.manual_seed(1000 * step + rank)  # noise and sigma of this update
        data = model.prepare_data_batch(batch_of(5, seed=100 * step + rank))
        result = trainer.training_step(model, scaler, data, iteration=step)
        loss = result.loss.detach().clone()
        dist.all_reduce(loss)
        return float(loss) / dist.get_world_size()

    if resume:
        loaded = checkpointer.load(model, model.optimizer_dict, model.scheduler_dict, scaler, path="latest")
        assert loaded.iteration == 2, loaded
    else:
        for step in range(2):
            update(step)
        checkpointer.save(model, model.optimizer_dict, model.scheduler_dict, scaler, iteration=2)
        checkpointer.finalize()
    loss = update(2)
    if rank == 0:
        torch.save({"loss": loss, "lr": optimizer.param_groups[0]["lr"]}, path)
    dist.barrier()
    dist.destroy_process_group()


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("mode", choices=["network", "train", "checkpoint", "autoregressive", "dmd"])
    parser.add_argument("output")
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--directory", default=None)
    parser.add_argument("--resume", action="store_true")
    args = parser.parse_args()
    torch.manual_seed(0)
    torch.set_num_threads(max(1, min(4, os.cpu_count() or 1)))
    if args.mode == "network":
        network_mode(args.output)
    elif args.mode == "train":
        train_mode(args.output, args.steps)
    elif args.mode == "autoregressive":
        autoregressive_mode(args.output)
    elif args.mode == "dmd":
        dmd_mode(args.output)
    else:
        checkpoint_mode(args.output, args.directory, args.resume)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
