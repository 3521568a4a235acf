"""Reference arm of the streaming benchmark (one GPU).

Runs the UNMODIFIED reference package (``baseline/_ref/wm``): ``Cosmos3Stream`` over a
``Cosmos3Network`` prepared by ``prepare_serving(network, cuda_graphs=True)`` — its Triton
generation-layer kernels, cuBLAS products and per-projection CUDA graphs
(``wm/inference/serving.py:51-84``, ``wm/networks/cosmos3/streaming.py:90-164``).  Same
workload as the other arm: batch 1, anchor ``[1, 48, 1, 30, 52]``, blocks of 4 latent frames
with 4 denoise steps at sigma (1.0, 0.75, 0.5, 0.25) and a commit, cache of 6 blocks plus
the anchor, top-aligned RoPE.  One untimed pass over ``--blocks`` blocks lets the Triton JIT
and the graph captures of every cache fill level happen first; the stream is then reset and
all ``--blocks`` blocks of the second pass are timed with CUDA events.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import traceback


def run(args: argparse.Namespace) -> dict:
    import torch

    from wm.codecs import Wan22VAECodec
    from wm.inference.serving import prepare_serving
    from wm.models.flow import rf_interpolate, rf_x0
    from wm.networks.cosmos3 import Cosmos3Conditioner, Cosmos3Config, build_network
    from wm.networks.cosmos3.network import Cosmos3Condition
    from wm.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_train import random_init_

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    config = Cosmos3Config(num_hidden_layers=args.layers)
    net = build_network(config, init_device="meta").to(torch.bfloat16).to_empty(device=device)
    net.initialize_after_materialization()
    random_init_(net, seed=0)
    net.eval().requires_grad_(False)
    cond = Cosmos3Conditioner(config=config, geometry_noise_sigma=0.0, init_device="meta",
                              codec=Wan22VAECodec(pretrained_path="unused", decoder=None))
    cond.to(torch.bfloat16).to_empty(device=device)
    random_init_(cond.text_encoder, seed=1)
    prepare_serving(net, cuda_graphs=not args.no_graphs)
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

    def one_pass(blocks: int) -> list[float]:
        stream.reset()
        stream.start(torch.randn((1, 48, 1, 30, 52), device=device, generator=g), condition(1))
        times = []
        for _ in range(blocks):
            cond_block = condition(4)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            clean = None
            for sigma in endpoints:
                s = torch.full((1,), sigma, device=device)
                noise = torch.randn(shape, device=device, generator=g)
                current = noise if clean is None else rf_interpolate(clean, noise, s)
                velocity = stream.denoise(current, s, cond_block)
                clean = rf_x0(current, s, velocity)
            stream.commit(clean, cond_block)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        return times

    with torch.inference_mode():
        warm = one_pass(min(args.blocks, 9))   # JIT + graph capture for every fill level
        times = one_pass(args.blocks)
    ordered = sorted(times)
    return {
        "metric": "Cosmos3Stream ms per 4-frame block (4 denoise + 1 commit)",
        "impl": "reference",
        "p50_ms": statistics.median(times),
        "p99_ms": ordered[min(len(ordered) - 1, int(0.99 * len(ordered)))],
        "mean_ms": statistics.fmean(times),
        "first_blocks_ms": times[:8], "warm_pass_first_blocks_ms": warm[:8],
        "blocks": args.blocks, "n_gpus": 1, "dtype": "bf16",
        "parallelism": "single GPU (the reference has no tensor parallelism)",
        "cuda_graphs": not args.no_graphs, "layers": args.layers,
        "cache": "anchor + 6 blocks (sink 1, history 24 frames), top-aligned RoPE",
        "tokens_per_block": 4 * 2 * 390,
        "timed": "all blocks of the second pass; the first pass warms JIT and graphs",
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--blocks", type=int, default=32)
    parser.add_argument("--layers", type=int, default=36)
    parser.add_argument("--no-graphs", action="store_true")
    args = parser.parse_args()
    try:
        line = run(args)
    except BaseException as error:
        if isinstance(error, KeyboardInterrupt):
            raise
        traceback.print_exc(file=sys.stderr)
        reason = f"{type(error).__name__}: {' '.join(str(error).split())[:300]}"
        line = {"impl": "reference", "unavailable": f"reference stream failed: {reason}"}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
