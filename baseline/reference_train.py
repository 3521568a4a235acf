"""Reference arm of the training benchmark.

Runs the UNMODIFIED reference package (``baseline/_ref/wm``) in a process whose import path
holds only that package and the two stand-ins under ``baseline/shims`` (``omegaconf`` and the
Transformer Engine multi-tensor Adam entry points); nothing of ``agentgarten_b200`` is
imported or loaded.  ``bench.py --impl reference`` replaces itself with this script.

The job is the reference's stock code path for the bidirectional recipe, built directly
instead of through the Hydra-composed recipe tree (Hydra is not installed):

* ``DiffusionModel(net=build_network(config, "meta"), conditioner=Cosmos3Conditioner(...))``
  with the recipe's ``ParallelConfig`` (bf16 parameters, FSDP2 per layer, selective
  activation checkpointing, per-method ``torch.compile``) and the frozen text tower's
  ``ParallelConfig`` (``wm/configs/experiments/cosmos3/bidirectional.py:16-34``);
* ``FusedAdam(lr=3e-5, betas=(0.9, 0.99), eps=1e-8, use_te_capturable_kernel=True,
  master_weights=True)`` and the ``LinearWarmup`` schedule
  (``wm/configs/experiments/cosmos3/__init__.py:136-145,181-183``);
* ``Trainer.training_step`` with a ``GradClip(max_norm=1.0)`` callback
  (``wm/infra/trainer.py:436-593``), ``torch`` runtime switches of ``wm/configs/base.py:22-30``.

Substitutions, all recorded in the printed line: synthetic cached latents and random
weights (as in the other arm), ``GradClip`` instead of ``GradClipMonitor`` (same clipping,
no spike diagnostics), the multi-tensor Adam stand-in, and ``compile=False`` only if Inductor
fails on this machine.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import traceback


def parse_args() -> argparse.Namespace:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=4)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--layers", type=int, default=36)
    parser.add_argument("--frames", type=int, default=21)
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--intermediate", type=int, default=12288)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--vocab", type=int, default=151936)
    parser.add_argument("--latent-hw", type=int, nargs=2, default=(30, 52))
    parser.add_argument("--text-tokens", type=int, default=512)
    parser.add_argument("--grad-accum", type=int, default=1)
    parser.add_argument("--recipe", default="bidirectional",
                        choices=["bidirectional", "ar_teacher_forcing", "ar_diffusion_forcing"])
    parser.add_argument("--device", default="cuda")
    parser.add_argument("--no-compile", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--dump-losses", default=None,
                        help="write the per-step losses to this JSON file (parity tests)")
    return parser.parse_args()


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc = index, None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, peak, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 7:
                continue
            try:
                clocks.append(float(cells[0]))
                peak = float(cells[1])
            except ValueError:
                continue
            for name, cell in zip(names, cells[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak,
                "samples": len(clocks), "reasons": sorted(reasons)}


def random_init_(module, seed: int, std: float = 0.02) -> None:
    """N(0, std) matrices and embeddings, unit norm weights, zero biases; sharded parameters
    are filled shard by shard."""
    import torch
    from torch.distributed.tensor import DTensor

    with torch.no_grad():
        generator = None
        for name, parameter in module.named_parameters():
            local = parameter.to_local() if isinstance(parameter, DTensor) else parameter
            if generator is None:
                generator = torch.Generator(device=local.device)
                generator.manual_seed(seed)
            if local.numel() == 0:
                continue
            if parameter.ndim >= 2:
                local.normal_(0.0, std, generator=generator)
            elif "norm" in name:
                local.fill_(1.0)
            elif name.endswith("bias"):
                local.zero_()
            else:
                local.normal_(0.0, std, generator=generator)


def build(args: argparse.Namespace, device, compile_layers: bool):
    import torch

    from wm.codecs import Wan22VAECodec
    from wm.infra.callbacks import CallbackGroup, GradClip
    from wm.infra.config import LazyCall
    from wm.infra.optim import FusedAdam, LinearWarmup
    from wm.infra.parallel import ParallelConfig
    from wm.infra.trainer import Trainer
    from wm.models.diffusion import DiffusionModel
    from wm.models.flow import RectifiedFlowSchedule
    from wm.networks.cosmos3 import Cosmos3Conditioner, Cosmos3Config, build_network

    config = Cosmos3Config(hidden_size=args.hidden, intermediate_size=args.intermediate,
                           num_hidden_layers=args.layers, num_attention_heads=args.heads,
                           num_key_value_heads=args.kv_heads, vocab_size=args.vocab)
    if args.vocab < 151_653:  # reduced vocabularies (CPU checks) cannot hold the released ids
        config.special_tokens = {"eos_token_id": 1, "start_of_generation": 2}
    dtype = "bfloat16" if device.type == "cuda" else "float32"
    parallel = ParallelConfig(parameter_dtype=dtype, fully_shard=True, context_parallel_size=1,
                              fsdp_mesh_shape=None, activation_checkpointing="selective",
                              compile=compile_layers)
    frozen = ParallelConfig(parameter_dtype=dtype, fully_shard=True, context_parallel_size=1,
                            fsdp_mesh_shape=None, activation_checkpointing="none", compile=False)
    # the codec object is lazy: with cached latents its weights are never read
    conditioner = Cosmos3Conditioner(
        config=config, codec=Wan22VAECodec(pretrained_path="unused-with-cached-latents",
                                           dtype="bfloat16", decoder=None),
        geometry_noise_sigma=0.0, init_device="meta")
    schedule = RectifiedFlowSchedule(shift=5.0, train_distribution="waver")
    if args.recipe == "bidirectional":
        model = DiffusionModel(
            net=build_network(config, init_device="meta"), conditioner=conditioner, schedule=schedule,
            text_dropout=0.1, parallel=parallel, conditioner_parallel=frozen,
            sampling={"num_steps": 35, "guidance": 6.0, "seed": 2026})
    else:
        # the autoregressive recipes of wm/configs/experiments/cosmos3/ar_*_forcing.py
        from wm.models.autoregressive import AutoregressiveModel

        forcing = args.recipe.removeprefix("ar_")
        model = AutoregressiveModel(
            net=build_network(config, init_device="meta"), conditioner=conditioner, mode=forcing,
            block_frames=4, schedule=schedule, text_dropout=0.1,
            corrupt_clean_history=forcing == "teacher_forcing", parallel=parallel,
            conditioner_parallel=frozen,
            sampling={"num_steps": 16, "guidance": 6.0, "seed": 2026, "sink_blocks": 0,
                      "recent_blocks": None})
    model.parallelize(device)
    random_init_(model.net, seed=0)
    random_init_(model.conditioner.text_encoder, seed=1)
    model.train()
    optimizer = FusedAdam(model._group_trainable_parameters(), lr=3e-5, betas=(0.9, 0.99), eps=1e-8,
                          weight_decay=0.0, adam_w_mode=True, use_te_capturable_kernel=True,
                          master_weights=True)
    scheduler = torch.optim.lr_scheduler.LambdaLR(
        optimizer, lr_lambda=LinearWarmup(warmup_steps=100, start_factor=0.1))
    model.optimizer_dict, model.scheduler_dict = {"net": optimizer}, {"net": scheduler}
    callbacks = CallbackGroup(
        {"trainer": {"callbacks": {"grad_clip": LazyCall(GradClip)(max_norm=1.0)}}}, trainer=None)
    trainer = Trainer(grad_accum_steps=args.grad_accum, callbacks=callbacks, device=device)
    grad_scaler = torch.amp.GradScaler(device=device.type, enabled=False)
    return config, model, trainer, grad_scaler


def synthetic_batch(config, args: argparse.Namespace, seed: int, pinned: bool):
    import torch

    g = torch.Generator().manual_seed(seed)
    shape = (1, config.latent_channels, args.frames, *args.latent_hw)
    batch = {
        "latent": torch.randn(shape, generator=g),
        "depth_latent": torch.randn(shape, generator=g),
        "normal_latent": torch.randn(shape, generator=g),
        "text_input_ids": torch.randint(min(1000, config.vocab_size // 2),
                                        min(config.vocab_size, 150000),
                                        (1, args.text_tokens), generator=g),
        "fps": torch.full((1,), 16.0),
    }
    if pinned:
        batch = {k: v.pin_memory() for k, v in batch.items()}
    return batch


def run(args: argparse.Namespace) -> dict:
    import torch
    import torch.distributed as dist

    from wm.infra import distributed

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    cuda = args.device == "cuda"
    device = distributed.init(device=args.device, backend="nccl" if cuda else "gloo")
    rank, world = distributed.get_rank(), distributed.get_world_size()
    if world != args.gpus and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} processes")
    # runtime switches of the base recipe
    torch.backends.cudnn.benchmark = True
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.set_float32_matmul_precision("high")
    torch._dynamo.config.recompile_limit = 32
    torch.fx.experimental._config.use_duck_shape = False
    torch.manual_seed(77 + rank)

    substitutions = ["synthetic cached latents and random-init weights",
                     "GradClip in place of GradClipMonitor",
                     "multi-tensor Adam of Transformer Engine replaced by torch._fused_adamw_ "
                     "on the FP32 masters plus a foreach copy"]
    compile_layers = cuda and not args.no_compile

    def sync() -> None:
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def make(compiled: bool):
        config, model, trainer, scaler = build(args, device, compiled)
        host = synthetic_batch(config, args, seed=1000 + rank, pinned=cuda)
        resident = {k: v.to(device) for k, v in host.items()}
        return config, model, trainer, scaler, host, resident

    iteration = 0
    losses: list[float] = []

    def step(model, trainer, scaler, batch, *, staged: bool):
        nonlocal iteration
        loss = None
        for micro in range(args.grad_accum):
            data = trainer._prepare_data_batch(model, batch) if staged \
                else model.prepare_data_batch(dict(batch))
            result = trainer.training_step(model, scaler, data, iteration=iteration,
                                           grad_accum_step=micro)
            loss = result.loss
        iteration += 1
        return loss

    config, model, trainer, scaler, host, resident = make(compile_layers)
    try:
        step(model, trainer, scaler, resident, staged=False)
    except torch.OutOfMemoryError:
        raise
    except Exception as error:  # Inductor / Triton failure on this machine
        if not compile_layers:
            raise
        flag = torch.tensor([1.0], device=device)
        note = f"{type(error).__name__}: {' '.join(str(error).split())[:200]}"
    else:
        flag, note = torch.tensor([0.0], device=device), None
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if compile_layers and float(flag) > 0:
        substitutions.append(f"compile=False (torch.compile failed: {note or 'on another rank'})")
        del model, trainer, scaler
        torch._dynamo.reset()
        if cuda:
            torch.cuda.empty_cache()
        compile_layers = False
        config, model, trainer, scaler, host, resident = make(False)
        step(model, trainer, scaler, resident, staged=False)

    warmup = max(args.warmup, 3)
    for _ in range(warmup - 1):
        losses.append(float(step(model, trainer, scaler, resident, staged=False)))
    sync()

    sampler = ClockSampler(device.index or 0) if cuda else None
    if sampler is not None and rank == 0:
        sampler.start()
    if cuda:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    import time

    sync()
    t0 = time.perf_counter()
    if cuda:
        start.record()
    for _ in range(args.steps):
        loss = step(model, trainer, scaler, resident, staged=False)
        if not cuda:
            losses.append(float(loss))
    if cuda:
        stop.record()
    sync()
    elapsed_ms = start.elapsed_time(stop) if cuda else (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if (sampler is not None and rank == 0) else {}
    loss_value = float(loss)

    e2e_ms = 0.0
    if not args.no_e2e:
        sync()
        t0 = time.perf_counter()
        if cuda:
            start.record()
        for _ in range(args.steps):
            loss_value = float(step(model, trainer, scaler, host, staged=True).item())
        if cuda:
            stop.record()
        sync()
        e2e_ms = start.elapsed_time(stop) if cuda else (time.perf_counter() - t0) * 1e3

    times = torch.tensor([elapsed_ms, e2e_ms], device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(times[0]), float(times[1])
    if args.dump_losses and rank == 0:
        with open(args.dump_losses, "w") as handle:
            json.dump(losses, handle)

    patch = config.patch_size
    tokens_per_clip = args.frames * (args.latent_hw[0] // patch) * (args.latent_hw[1] // patch)
    tokens = tokens_per_clip * world * args.steps * args.grad_accum
    line = {
        "metric": "train latent-tokens/s/box (bidirectional rectified flow)" if args.recipe == "bidirectional"
                  else f"train latent-tokens/s/box ({args.recipe})",
        "value": tokens / (elapsed_ms / 1e3),
        "unit": "latent RGB tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": elapsed_ms / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16" if cuda else "fp32",
        "data": "synthetic cached latents N(0,1), random-init weights",
        "impl": "reference",
        "config": {
            "model": f"Cosmos3-Nano-shaped DiT: {config.num_hidden_layers} layers, hidden "
                     f"{config.hidden_size}, {config.num_attention_heads}/"
                     f"{config.num_key_value_heads} heads x {config.head_dim}, MLP "
                     f"{config.intermediate_size}, plus frozen text tower of the same size",
            "global_batch": world,
            "seq_len": tokens_per_clip,
            "tokens_in_sequence": 2 * tokens_per_clip,
            "latent": [1, config.latent_channels, args.frames, *args.latent_hw],
            "parallelism": f"dp{world} (FSDP2 per layer, bf16 parameters, FP32 reduce, selective "
                           f"activation checkpointing, torch.compile={compile_layers})",
            "grad_accum_steps": args.grad_accum,
            "optimizer": "Adam lr 3e-5 betas (0.9, 0.99), FP32 master, grad clip 1.0",
            "l2_policy": "inputs larger than L2 (14 GB of weights stream every step)",
        },
        "clocks": clocks,
        "loss": loss_value,
        "substitutions": substitutions,
        "peak_memory_gb": round(torch.cuda.max_memory_allocated(device) / 2 ** 30, 1) if cuda else None,
    }
    if not args.no_e2e:
        line["e2e"] = {
            "value": tokens / (e2e_ms / 1e3),
            "unit": "latent RGB tokens/s",
            "ms_per_step": e2e_ms / args.steps,
            "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in host.values())
            * args.grad_accum,
            "d2h_bytes_per_step": 4,
        }
    if world > 1:
        dist.destroy_process_group()
    return line if rank == 0 else {}


def main() -> int:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    try:
        line = run(args)
    except BaseException as error:  # every failure becomes the "unavailable" line
        if isinstance(error, (KeyboardInterrupt,)):
            raise
        if rank == 0:
            reason = f"{type(error).__name__}: {' '.join(str(error).split())[:300]}"
            if not isinstance(error, SystemExit):
                traceback.print_exc(file=sys.stderr)
            print(json.dumps({"impl": "reference", "n_gpus": args.gpus,
                              "unavailable": f"reference run failed at {args.gpus} GPU(s): {reason}"}))
        return 0
    if rank == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
