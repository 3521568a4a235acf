"""Worker for the multi-GPU tests; launched by torch.distributed.run, one rank per GPU."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from agentgarten_b200.infra import distributed  # noqa: E402
from agentgarten_b200.infra.optim import FusedAdam  # noqa: E402


def check_sharded_adam(device, rank, world):
    shapes = [(64, 32), (7, 24), (130,), (3, 5, 8), (1, 16)]
    torch.manual_seed(0)  # same parameters everywhere
    base = [torch.randn(s, device=device).to(torch.bfloat16) for s in shapes]
    sharded = [torch.nn.Parameter(b.clone()) for b in base]
    plain = [torch.nn.Parameter(b.clone()) for b in base]
    opt = FusedAdam(sharded, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01,
                    use_te_capturable_kernel=True, master_weights=True)
    ref = FusedAdam(plain, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01,
                    use_te_capturable_kernel=True, master_weights=True, flat=False,
                    process_group=None)
    assert opt.engine is not None and opt.engine.world == world
    for step in range(3):
        grads_all = []
        for r in range(world):
            g = torch.Generator(device=device).manual_seed(100 * step + r)
            grads_all.append([torch.randn(s, device=device, generator=g).to(torch.bfloat16) for s in shapes])
        for p, g in zip(sharded, grads_all[rank]):
            p.grad.copy_(g)
        mean = [torch.stack([grads_all[r][i].float() for r in range(world)]).sum(0) / world
                for i in range(len(shapes))]
        for q, g in zip(plain, mean):
            q.grad = g.to(torch.bfloat16)
        expected_sq = torch.stack([g.square().sum() for g in mean]).sum()
        got = opt.grad_norm_sq()
        assert torch.allclose(got, expected_sq, rtol=1e-3), (float(got), float(expected_sq))
        opt.step()
        # the reference optimizer must not all-reduce: its gradients are already the mean
        ref._reduced = True
        ref.step()
        opt.zero_grad()
        ref.zero_grad()
        torch.cuda.synchronize()
        for p, q in zip(sharded, plain):
            assert torch.allclose(p.float(), q.float(), atol=2e-2, rtol=2e-2), step
    # every rank must hold identical parameters (the all-gather half of the Adam kernel)
    flat = opt.engine.flat_param.float()
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    for other in gathered:
        assert torch.equal(other, gathered[0])


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    device = distributed.init(device="cuda", backend="nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    check_sharded_adam(device, rank, world)
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
