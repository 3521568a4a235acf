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

    from agentgarten_b200.bench_support import stream_benchmark
    from agentgarten_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    rank = dist.get_rank() if world > 1 else 0
    native.require()
    result = stream_benchmark(device, blocks=args.blocks, layers=args.layers, graphs=not args.no_graphs,
                              tensor_parallel=args.tensor_parallel, trace=args.trace)
    if rank == 0:
        phases = result.pop("phase_ms", None)
        if phases is not None:
            print("phase ms (mean per call, rank 0):", json.dumps(phases))
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
