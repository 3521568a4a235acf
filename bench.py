"""Headline benchmark: bidirectional rectified-flow training of the Cosmos3-Nano-shaped DiT.

``python bench.py --gpus N --steps K --warmup W`` (under torchrun for N > 1) trains on
synthetic cached latents ``[1, 48, 21, 30, 52]`` (+ depth and normal latents of the same
shape, 512 prompt tokens through the frozen text tower) with random-initialised weights,
one clip per GPU (weak scaling), bf16 parameters/activations with FP32 master weights and
Adam moments, gradient clipping and one optimizer update per step.  It prints one JSON line
with the whole-job throughput in latent RGB tokens per second.

Two timed regions, both with CUDA events on the compute stream, max over ranks:
``value`` keeps the batch resident on the device; ``e2e`` additionally copies every step's
batch from pinned host memory and reads the loss back to the host.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = os.path.join(ROOT, "baseline", "_ref")
REFERENCE_SHIMS = os.path.join(ROOT, "baseline", "shims")
REFERENCE_RUNNER = os.path.join(ROOT, "baseline", "reference_train.py")


def parse_args() -> argparse.Namespace:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=4)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="agentgarten_b200", choices=["agentgarten_b200", "reference"])
    parser.add_argument("--layers", type=int, default=36, help="smaller values are for debugging only")
    parser.add_argument("--frames", type=int, default=None,
                        help="latent frames per clip (default 21; 61 for the autoregressive recipes)")
    parser.add_argument("--recipe", default="bidirectional",
                        choices=["bidirectional", "ar_diffusion_forcing", "ar_teacher_forcing"],
                        help="the headline metric is the default; the others measure the other recipes")
    parser.add_argument("--context-parallel", type=int, default=1,
                        help="ranks that share one clip (divides --gpus); 1 = data parallel only")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--grad-accum", type=int, default=1,
                        help="microbatches per optimizer update (the headline uses 1)")
    parser.add_argument("--no-stream", action="store_true",
                        help="skip the streaming measurement that follows the training regions")
    parser.add_argument("--stream-blocks", type=int, default=32)
    parser.add_argument("--reference-args", default="",
                        help="extra arguments for baseline/reference_train.py (debugging)")
    return parser.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while timing."""

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


def reference_environment() -> dict[str, str]:
    """Environment of the reference process: its import path holds the unmodified reference
    package and the stand-ins for its two missing dependencies, nothing of this package."""
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join((REFERENCE_ROOT, REFERENCE_SHIMS))
    env.pop("PYTHONSTARTUP", None)
    return env


def run_reference(args: argparse.Namespace) -> int:
    """Replaces this process with ``baseline/reference_train.py`` (one per rank, so the
    launcher's RANK / WORLD_SIZE / MASTER_* reach it unchanged)."""
    reason = None
    if not os.path.isfile(os.path.join(REFERENCE_ROOT, "wm", "__init__.py")):
        reason = ("the reference package is not installed under baseline/_ref "
                  "(copy the reference's wm/ directory there)")
    elif args.context_parallel != 1:
        reason = "the reference arm runs the recipes data-parallel only (no context parallelism)"
    if reason is not None:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": reason}))
        return 0
    command = [sys.executable, REFERENCE_RUNNER, "--gpus", str(args.gpus), "--steps", str(args.steps),
               "--warmup", str(args.warmup), "--layers", str(args.layers),
               "--frames", str(args.frames or (21 if args.recipe == "bidirectional" else 61)),
               "--grad-accum", str(args.grad_accum), "--recipe", args.recipe]
    if args.no_e2e:
        command.append("--no-e2e")
    if args.reference_args:
        command.extend(args.reference_args.split())
    sys.stdout.flush()
    os.chdir(os.path.join(ROOT, "baseline"))
    os.execve(sys.executable, command, reference_environment())
    return 0  # not reached


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from agentgarten_b200.bench_support import batch_bytes, build_training_job, synthetic_batch
    from agentgarten_b200.infra import distributed
    from agentgarten_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} processes "
                             f"(WORLD_SIZE={world})")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    device = distributed.init(device="cuda", backend="nccl")
    rank = distributed.get_rank()
    native.require()

    frames = args.frames or (21 if args.recipe == "bidirectional" else 61)
    cp = args.context_parallel
    if cp < 1 or world % cp:
        raise SystemExit(f"--context-parallel {cp} does not divide {world} ranks")
    job = build_training_job(device, layers=args.layers, frames=frames, recipe=args.recipe,
                             context_parallel=cp)
    job.grad_accum_steps = max(1, args.grad_accum)
    # the ranks that share a clip get the same batch and draw the same noise
    host_batch = synthetic_batch(job, "cpu", seed=1000 + rank // cp, pinned=True)
    torch.manual_seed(77 + rank // cp)
    device_batch = {k: v.to(device) for k, v in host_batch.items()}

    def to_device(batch):
        return {k: v.to(device, non_blocking=True) for k, v in batch.items()}

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        job.step(device_batch)
    barrier()

    # ------------------------------------------------------------ device-resident region
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()
    launches_before = native.launches()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        loss = job.step(device_batch)
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    launches = native.launches() - launches_before
    clocks = sampler.stop() if rank == 0 else {}
    loss_value = float(loss)

    # ---------------------------------------------------------------- end-to-end region
    e2e_ms = None
    if not args.no_e2e:
        barrier()
        start.record()
        for _ in range(args.steps):
            loss_value = float(job.step(host_batch, stage=to_device).item())  # device -> host read
        stop.record()
        barrier()
        e2e_ms = start.elapsed_time(stop)

    times = torch.tensor([elapsed_ms, e2e_ms if e2e_ms is not None else 0.0], device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_max = float(times[0]), float(times[1])
    status = int(native.ext().status(device.index or 0).item())

    # Every rank must hold the same parameters after the timed updates (the all-gather half of
    # the optimizer kernel writes them through peer memory): checksum, min and max over ranks.
    flat = job.optimizer.engine.flat_param.view(torch.int16)
    sums = torch.zeros(2, dtype=torch.int64, device=device)
    for chunk in flat.split(1 << 26):          # bit patterns, in pieces: no 50 GB temporaries
        wide = chunk.to(torch.int64)
        sums[0] += wide.sum()
        sums[1] += (wide * wide).sum()
    low, high = sums.clone(), sums.clone()
    if world > 1:
        dist.all_reduce(low, op=dist.ReduceOp.MIN)
        dist.all_reduce(high, op=dist.ReduceOp.MAX)
    replicas_in_sync = bool(torch.equal(low, high)) if cp == 1 else None
    peak_gb = round(torch.cuda.max_memory_allocated(device) / 2 ** 30, 1)
    rgb_tokens, accum, model_config = job.rgb_tokens_per_clip, job.grad_accum_steps, job.config
    latent_hw, job_frames = job.latent_hw, job.frames

    # Streaming (the second half of the headline metric): the training job is released first.
    stream = None
    if not args.no_stream and args.recipe == "bidirectional" and args.layers == 36:
        import gc

        from agentgarten_b200.bench_support import stream_benchmark

        del job, device_batch, flat, loss
        gc.collect()
        torch.cuda.empty_cache()
        try:
            result = stream_benchmark(device, blocks=args.stream_blocks)
            stream = {k: result[k] for k in ("p50_ms", "p99_ms", "mean_ms", "blocks", "n_gpus",
                                             "parallelism", "cuda_graphs", "kernel_status", "timed")}
        except Exception as error:  # the training numbers stand on their own
            stream = {"unavailable": f"{type(error).__name__}: {' '.join(str(error).split())[:200]}"}

    if rank == 0:
        tokens = rgb_tokens * (world // cp) * args.steps * accum
        value = tokens / (elapsed_ms / 1e3)
        line = {
            "metric": "train latent-tokens/s/box (bidirectional rectified flow)"
            if args.recipe == "bidirectional" else f"train latent-tokens/s/box ({args.recipe})",
            "value": value,
            "unit": "latent RGB tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic cached latents N(0,1), random-init weights",
            "impl": "agentgarten_b200",
            "config": {
                "model": f"Cosmos3-Nano-shaped DiT: {model_config.num_hidden_layers} layers, hidden "
                         f"{model_config.hidden_size}, {model_config.num_attention_heads}/"
                         f"{model_config.num_key_value_heads} heads x {model_config.head_dim}, MLP "
                         f"{model_config.intermediate_size}, plus frozen text tower of the same size",
                "global_batch": world // cp,
                "seq_len": rgb_tokens,
                "tokens_in_sequence": 2 * rgb_tokens,
                "latent": [1, 48, job_frames, *latent_hw],
                "parallelism": f"dp{world // cp}" + (f" x cp{cp} (Ulysses)" if cp > 1 else "") +
                               " (replicated bf16 parameters, sharded FP32 optimizer state, "
                               "peer-memory reduce-scatter under the backward pass + Adam + all-gather)",
                "grad_accum_steps": accum,
                "optimizer": "Adam lr 3e-5 betas (0.9, 0.99), FP32 master, grad clip 1.0",
                "l2_policy": "inputs larger than L2 (14 GB of weights stream every step)",
            },
            "clocks": clocks,
            "gpu_launches": launches,
            "loss": loss_value,
            "kernel_status": status,
            "peak_memory_gb": peak_gb,
            "replicas_in_sync": replicas_in_sync,
        }
        if stream is not None:
            line["stream"] = stream
        if e2e_ms is not None:
            line["e2e"] = {
                "value": tokens / (e2e_max / 1e3),
                "unit": "latent RGB tokens/s",
                "ms_per_step": e2e_max / args.steps,
                "h2d_bytes_per_step": batch_bytes(host_batch) * accum,
                "d2h_bytes_per_step": 4,
            }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
