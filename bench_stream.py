"""Streaming-inference benchmark: Cosmos3Stream, batch 1, bf16, CUDA graphs.

Anchor ``[1, 48, 1, 30, 52]``, then ``--blocks`` blocks of 4 latent frames, each with fresh
depth/normal latents, 4 denoise steps at the sigma endpoints (1.0, 0.75, 0.5, 0.25) followed
by a commit into a bounded cache of 6 blocks plus the anchor.  Prints one JSON line with the
p50 / p99 milliseconds per block (device time, CUDA events around each block) over ALL
``--blocks`` blocks: a first, untimed pass over nine blocks captures the CUDA graph of every
cache fill level, then the stream is reset and the timed pass starts from a fresh anchor.

``--impl reference`` runs the unmodified reference package on one GPU through
``baseline/reference_stream.py`` (same workload, its own kernels and graphs).

On several GPUs (``python -m torch.distributed.run --nproc-per-node N ... bench_stream.py``)
the tower is tensor parallel over the ranks: every rank feeds the same seeded inputs, the
per-block time is the maximum over ranks.  ``--tensor-parallel`` selects the tensor-parallel
kernels on one GPU as well.
"""

from __future__ import annotations

import argparse
import json
import statistics


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--blocks", type=int, default=32)
    parser.add_argument("--layers", type=int, default=36)
    parser.add_argument("--no-graphs", action="store_true")
    parser.add_argument("--tensor-parallel", action="store_true")
    parser.add_argument("--trace", action="store_true",
                        help="eager run with per-phase CUDA events of the tensor-parallel layers")
    parser.add_argument("--impl", default="agentgarten_b200", choices=["agentgarten_b200", "reference"])
    args = parser.parse_args()

    import os
    import sys

    if args.impl == "reference":
        root = os.path.dirname(os.path.abspath(__file__))
        if not os.path.isfile(os.path.join(root, "baseline", "_ref", "wm", "__init__.py")):
            print(json.dumps({"impl": "reference", "unavailable":
                              "the reference package is not installed under baseline/_ref"}))
            return 0
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "the reference streams on one GPU only (it has no tensor parallelism)"}))
            return 0
        env = dict(os.environ)
        env["PYTHONPATH"] = os.pathsep.join((os.path.join(root, "baseline", "_ref"),
                                             os.path.join(root, "baseline", "shims")))
        command = [sys.executable, os.path.join(root, "baseline", "reference_stream.py"),
                   "--blocks", str(args.blocks), "--layers", str(args.layers)]
        if args.no_graphs:
            command.append("--no-graphs")
        sys.stdout.flush()
        os.chdir(os.path.join(root, "baseline"))
        os.execve(sys.executable, command, env)

    import torch
    import torch.distributed as dist

    from agentgarten_b200.bench_support import random_init_
    from agentgarten_b200.inference.serving import prepare_serving
    from agentgarten_b200.models.flow import rf_interpolate, rf_x0
    from agentgarten_b200.networks.cosmos3 import Cosmos3Config, build_network
    from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
    from agentgarten_b200.networks.cosmos3.network import Cosmos3Condition
    from agentgarten_b200.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy
    from agentgarten_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    rank = dist.get_rank() if world > 1 else 0
    native.require()
    config = Cosmos3Config(num_hidden_layers=args.layers)
    net = build_network(config, init_device="meta").to(torch.bfloat16).to_empty(device=device)
    random_init_(net, seed=0)
    cond = Cosmos3Conditioner(config=config, codec=None, init_device="meta", geometry_noise_sigma=0.0)
    cond.to(torch.bfloat16).to_empty(device=device)
    random_init_(cond.text_encoder, seed=1)
    sharded = world > 1 or args.tensor_parallel
    if args.trace:
        args.no_graphs = True
    prepare_serving(net, cuda_graphs=not args.no_graphs, tensor_parallel=True if sharded else None,
                    max_tokens=4096)
    policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=24, rope="top_aligned",
                          train_frames=61)
    g = torch.Generator(device=device).manual_seed(0)
    shape = (1, 48, 4, 30, 52)
    ids = torch.randint(1000, 150000, (1, 512), device=device, generator=g)
    with torch.inference_mode():
        text = cond.text_encoder(ids, None)

    def condition(frames):
        s = (1, 48, frames, 30, 52)
        return Cosmos3Condition(text=text, depth=torch.randn(s, device=device, generator=g),
                                normal=torch.randn(s, device=device, generator=g),
                                fps=torch.full((1,), 16.0, device=device))

    endpoints = (1.0, 0.75, 0.5, 0.25)
    stream = Cosmos3Stream(net, policy)
    anchor = torch.randn((1, 48, 1, 30, 52), device=device, generator=g)
    # every fill-level graph is captured here, before the timed blocks
    stream.capture_graphs(anchor, condition(1), condition(4))
    stream.start(anchor, condition(1))
    times = []
    launches_before = native.launches()
    for block in range(args.blocks):
        if args.trace and sharded and block == args.blocks - 2:
            net._tensor_parallel.trace = {}
        cond_block = condition(4)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        clean = None
        for step, sigma in enumerate(endpoints):
            s = torch.full((1,), sigma, device=device)
            noise = torch.randn(shape, device=device, generator=g)
            current = noise if clean is None else rf_interpolate(clean, noise, s)
            velocity = stream.denoise(current, s, cond_block)
            clean = rf_x0(current, s, velocity)
        stream.commit(clean, cond_block)
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
        # A bounded wait that ran out on any rank ends the run on all of them: the remaining
        # blocks would only repeat the failure.  (Outside the timed region.)
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
    if args.trace and sharded and rank == 0:
        print("phase ms (mean per call, rank 0):", json.dumps(net._tensor_parallel.trace_summary()))
    if rank != 0:
        dist.destroy_process_group()
        return 0
    steady = times  # all blocks count: the graphs were captured before the first one
    steady_sorted = sorted(steady)
    print(json.dumps({
        "metric": "Cosmos3Stream ms per 4-frame block (4 denoise + 1 commit)",
        "p50_ms": statistics.median(steady),
        "p99_ms": steady_sorted[min(len(steady_sorted) - 1, int(0.99 * len(steady_sorted)))],
        "first_blocks_ms": times[:8], "blocks": args.blocks, "n_gpus": world, "dtype": "bf16",
        "parallelism": f"tp{world} (heads and MLP columns; GEMM+reduce-scatter / all-gather+GEMM over peer memory)"
        if sharded else "single GPU",
        "cuda_graphs": not args.no_graphs, "layers": args.layers,
        "cache": "anchor + 6 blocks (sink 1, history 24 frames), top-aligned RoPE",
        "tokens_per_block": 4 * 2 * 390, "gpu_launches": native.launches() - launches_before,
        "kernel_status": status,
    }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
