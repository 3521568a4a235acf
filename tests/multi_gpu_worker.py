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


def check_overlapped_gradient_path(device, rank, world):
    """Two updates of a small job with per-rank data: reducing each layer's gradients from its
    backward pass (side stream, counters between the ranks) gives bit for bit the parameters of
    the run that reduces everything after the backward pass, on every rank."""
    from agentgarten_b200.bench_support import build_training_job, synthetic_batch
    from agentgarten_b200.ops import native

    results = {}
    for mode in ("1", "0"):
        os.environ["AGB200_GRAD_OVERLAP"] = mode
        job = build_training_job(device, layers=3, hidden=512, intermediate=1024, heads=4, kv_heads=2,
                                 frames=3, latent_hw=(16, 16), text_tokens=20)
        batch = synthetic_batch(job, device, seed=500 + rank)
        torch.manual_seed(9 + rank)
        for _ in range(2):
            job.step(batch)
        torch.cuda.synchronize()
        engine = job.optimizer.engine
        results[mode] = (engine.flat_param.clone(), len(engine._buckets))
        assert int(native.ext().status(device.index).item()) == 0, "a bounded wait gave up"
        del job, engine
    os.environ.pop("AGB200_GRAD_OVERLAP")
    assert results["1"][1] >= 3, results["1"][1]      # one bucket per layer plus the rest
    assert results["0"][1] == 1
    assert torch.equal(results["1"][0], results["0"][0])
    gathered = [torch.empty_like(results["1"][0]) for _ in range(world)]
    dist.all_gather(gathered, results["1"][0])
    assert all(torch.equal(other, gathered[0]) for other in gathered)  # replicas agree


def check_tensor_parallel_stream(device, rank, world):
    """Sharded serving over peer memory against the single-GPU layer path, eager and replayed."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network

    from agentgarten_b200.inference.serving import prepare_serving, release_serving
    from agentgarten_b200.networks.cosmos3.network import Cosmos3Condition
    from agentgarten_b200.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy
    from agentgarten_b200.ops import native

    config = tiny_config(hidden_size=512, intermediate_size=1024, num_attention_heads=8,
                         num_key_value_heads=world, head_dim=128, mrope_section=(24, 20, 20))
    net = tiny_network(config, device="cpu", seed=0).to(device, torch.bfloat16).eval()
    cond = tiny_conditioner(config, device="cpu", seed=1).to(device, torch.bfloat16)
    batch = {k: v.to(device) for k, v in synthetic_batch(frames=17, height=8, width=12, text=9, seed=5).items()}
    encoded = cond.encode(batch, training=False)
    condition, latent = cond.condition(encoded), encoded["latent"]
    policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, rope="top_aligned", train_frames=13)

    def block(lo, hi):
        return Cosmos3Condition(text=condition.text, depth=condition.depth[:, :, lo:hi],
                                normal=condition.normal[:, :, lo:hi], fps=condition.fps)

    def rollout(**serving):
        prepare_serving(net, **serving)
        stream = Cosmos3Stream(net, policy)
        stream.start(latent[:, :, :1], block(0, 1))
        outs = []
        gen = torch.Generator(device=device).manual_seed(3)
        for b in range(4):
            lo, hi = 1 + 4 * b, 5 + 4 * b
            noisy = torch.randn(latent[:, :, lo:hi].shape, device=device, generator=gen)
            for sigma in (1.0, 0.5):
                outs.append(stream.denoise(noisy, torch.tensor([sigma], device=device), block(lo, hi)))
            stream.commit(latent[:, :, lo:hi], block(lo, hi))
        torch.cuda.synchronize()
        return outs

    plain = rollout(cuda_graphs=False)
    eager = rollout(cuda_graphs=False, tensor_parallel=True, max_tokens=1024)
    replay = rollout(cuda_graphs=True, tensor_parallel=True, max_tokens=1024)
    assert int(native.ext().status(device.index).item()) == 0, "a bounded wait gave up"
    for a, b, c in zip(plain, eager, replay):
        assert torch.isfinite(b).all()
        error = float((b.float() - a.float()).norm() / a.float().norm())
        assert error < 2e-2, error
        assert torch.equal(b, c)
        same = [torch.empty_like(b) for _ in range(world)]
        dist.all_gather(same, b.contiguous())
        assert all(torch.equal(other, same[0]) for other in same)  # every rank holds all rows
    release_serving(net)


def check_context_parallel_training(device, rank, world):
    """Ulysses context parallelism over NCCL with the CUDA kernels: same loss and the same
    summed gradients as the unsharded model on the same clip."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network

    from agentgarten_b200.models.diffusion import DiffusionModel
    from agentgarten_b200.parallel.engine import ParallelConfig

    config = tiny_config(hidden_size=512, intermediate_size=1024, num_attention_heads=8,
                         num_key_value_heads=2 * world, head_dim=128, mrope_section=(24, 20, 20))
    losses, grads = {}, {}
    for cp in (1, world):
        parallel = ParallelConfig(parameter_dtype="bfloat16", context_parallel_size=cp,
                                  fully_shard=False, activation_checkpointing="none")
        frozen = ParallelConfig(parameter_dtype="bfloat16", fully_shard=False, activation_checkpointing="none")
        model = DiffusionModel(net=tiny_network(config, seed=0), conditioner=tiny_conditioner(config, seed=1),
                               text_dropout=0.0, parallel=parallel, conditioner_parallel=frozen)
        model.parallelize(device)
        raw = {k: v.to(device) for k, v in synthetic_batch(frames=5, height=16, width=16, text=9, seed=3).items()}
        batch = model.prepare_data_batch(raw)
        torch.manual_seed(11)
        model.train()
        _, loss = model.training_step(batch, 0)
        loss.backward()
        losses[cp] = float(loss)
        grads[cp] = {n: p.grad.float().clone() for n, p in model.net.named_parameters() if p.grad is not None}
    assert abs(losses[1] - losses[world]) < 2e-2 * max(1.0, abs(losses[1])), losses
    worst = 0.0
    for name, full in grads[1].items():
        part = grads[world][name].clone()
        dist.all_reduce(part)
        scale = float(full.norm()) + 1e-6
        err = min(float((part - full).norm()), float((part / world - full).norm())) / scale
        worst = max(worst, err)
    assert worst < 5e-2, worst


def check_peer_exchange(device, rank, world):
    """The peer-memory all-to-all against the library collective: several sizes (one of them
    larger than the first buffer, so that it grows), repeated so that both halves of the
    receive buffer and the monotonic counters are reused."""
    from agentgarten_b200.parallel import peer_exchange

    group = dist.group.WORLD
    torch.manual_seed(100 + rank)
    for shape in ((world, 3, 40, 128), (world, 1, 8, 64), (world, 20000, 8, 128), (world, 3, 40, 128)):
        for repeat in range(5):
            value = torch.randn(shape, device=device).bfloat16()
            want = torch.empty_like(value)
            dist.all_to_all_single(want, value, group=group)
            got = peer_exchange.exchange(value, group)
            assert got is not None, "the peer path must apply to an NCCL group on one node"
            assert torch.equal(got, want), (shape, repeat)
    torch.cuda.synchronize()
    from agentgarten_b200.ops import native
    assert int(native.ext().status(device.index).item()) == 0
    dist.barrier()
    peer_exchange.release()


def check_switch_consensus(device, rank, world):
    """The maximum of a few small values over the ranks through the NVSwitch multicast mapping
    against the library all-reduce, repeated so that both halves of the buffer and the call
    counter are reused; where the GPUs have no multicast mapping the same call takes the library
    path and must agree all the same."""
    from agentgarten_b200.ops import native
    from agentgarten_b200.parallel import consensus

    for call in range(7):
        word = torch.tensor([float((rank + call) % 3 == 0), float((call * (rank + 1)) % 8), float(rank)],
                            device=device)
        want = word.clone()
        dist.all_reduce(want, op=dist.ReduceOp.MAX)
        got = consensus.maximum(word.clone())
        assert torch.equal(got, want), (call, got.tolist(), want.tolist())
    torch.cuda.synchronize()
    assert int(native.ext().status(device.index).item()) == 0
    # the trainer's consensus takes the same path: one rank with a non-finite gradient stops all
    from agentgarten_b200.infra.nonfinite import synchronize_found_nonfinite

    for bad_rank in (None, world - 1):
        weight = torch.nn.Parameter(torch.ones(8, device=device))
        weight.grad = torch.ones(8, device=device)
        if rank == bad_rank:
            weight.grad[3] = float("inf")
        verdict = synchronize_found_nonfinite(None, (torch.optim.SGD([weight], lr=0.1),), fallback_device=device)
        assert verdict == (bad_rank is not None), (bad_rank, verdict)
    used = consensus._link(dist.group.WORLD, device) is not None
    if rank == 0:
        print("SWITCH_CONSENSUS", "multimem" if used else "library path (no multicast mapping)")
    dist.barrier()
    consensus.release()


def check_switch_share(device, rank, world):
    """All-gather and broadcast through multicast stores against the library collectives: sizes
    that are no multiple of 16 bytes, one that makes the buffer grow, repeated calls that reuse
    both halves; then the context-parallel gather (values and gradient) on that path."""
    from agentgarten_b200.ops import native
    from agentgarten_b200.parallel import switch_share

    g = torch.Generator(device=device).manual_seed(100 + rank)
    used = None
    for call, shape in enumerate([(1, 37, 5), (2, 300, 64), (1, 2048, 4096), (3, 7), (1, 2048, 4096),
                                  (3 << 20, 5)]):
        dtype = (torch.bfloat16, torch.float32)[call % 2]
        value = torch.randn(shape, device=device, generator=g).to(dtype)
        parts = [torch.empty_like(value) for _ in range(world)]
        dist.all_gather(parts, value)
        got = switch_share.all_gather(value)
        used = got is not None
        if used:
            assert torch.equal(got, torch.stack(parts)), (call, shape)
        payload = (value.float() * 3).to(dtype).view(torch.uint8).reshape(-1)[: value.numel() * 2 - 3]
        payload = payload.clone()
        want = payload.clone()
        source = call % world
        dist.broadcast(want, src=source)
        if switch_share.broadcast(payload, source):
            assert torch.equal(payload, want), (call, shape)
    torch.cuda.synchronize()
    assert int(native.ext().status(device.index).item()) == 0
    from agentgarten_b200.networks.cosmos3.context_parallel import _Gather

    local = torch.randn(2, 11, 24, device=device, generator=g, requires_grad=True)
    whole = _Gather.apply(local, dist.group.WORLD, rank, world)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.detach())
    assert torch.equal(whole, torch.cat(parts, dim=1))
    weight = torch.randn(whole.shape, device=device, generator=torch.Generator(device=device).manual_seed(7))
    (whole * weight).sum().backward()
    assert torch.equal(local.grad, weight[:, rank * 11:(rank + 1) * 11] * world)
    if rank == 0:
        print("SWITCH_SHARE", "multimem" if used else "library path (no multicast mapping)")
    dist.barrier()
    switch_share.release()


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    device = distributed.init(device="cuda", backend="nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    checks = [check_sharded_adam, check_overlapped_gradient_path, check_tensor_parallel_stream,
              check_context_parallel_training, check_peer_exchange, check_switch_consensus, check_switch_share]
    wanted = sys.argv[1:]   # names of checks to run; all of them without arguments
    for check in checks:
        if wanted and check.__name__ not in wanted:
            continue
        check(device, rank, world)
        dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
