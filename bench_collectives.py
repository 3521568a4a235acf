"""All-gather and broadcast through NVSwitch multicast stores against the NCCL collectives.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench_collectives.py [--sizes-mb 0.25 2 16 64]

Each size is the payload per rank.  Both paths are timed with CUDA events over 20 calls after 5
warm-up calls, bracketed by a barrier and a device synchronise; the figure is the maximum over the
ranks.  The package's path includes the allocation of its output, as a caller sees it.  Rank 0
prints one JSON line per size.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from agentgarten_b200.infra import distributed
from agentgarten_b200.parallel import switch_share


def _timed(call, device, repeats: int = 20, warmup: int = 5) -> float:
    for _ in range(warmup):
        call()
    torch.cuda.synchronize(device)
    dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        call()
    stop.record()
    torch.cuda.synchronize(device)
    slowest = torch.tensor([start.elapsed_time(stop) / repeats], device=device)
    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    return float(slowest) * 1000.0


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--sizes-mb", type=float, nargs="+", default=[0.25, 2.0, 16.0, 64.0])
    args = parser.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    device = distributed.init(device="cuda", backend="nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    for size in args.sizes_mb:
        count = int(size * (1 << 20)) // 2
        value = torch.randn(count, device=device).to(torch.bfloat16)
        room = torch.empty(world * count, dtype=torch.bfloat16, device=device)
        payload = torch.empty(2 * count, dtype=torch.uint8, device=device)
        on_switch = switch_share.all_gather(value) is not None
        row = {
            "mb_per_rank": size, "n_gpus": world, "path": "multimem" if on_switch else "library",
            "all_gather_us": _timed(lambda: switch_share.all_gather(value), device) if on_switch else None,
            "all_gather_nccl_us": _timed(lambda: dist.all_gather_into_tensor(room, value), device),
            "broadcast_us": _timed(lambda: switch_share.broadcast(payload, 0), device) if on_switch else None,
            "broadcast_nccl_us": _timed(lambda: dist.broadcast(payload, src=0), device),
        }
        if rank == 0:
            print(json.dumps(row), flush=True)
    dist.barrier()
    switch_share.release()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
