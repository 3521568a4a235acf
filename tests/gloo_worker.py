"""Worker for the CPU multi-rank tests: ``torchrun ... tests/gloo_worker.py <case> [args]``.

Failures are injected on the host only: a dataset iterator that raises on one rank, an
iterator that ends early on one rank, an unpicklable batch.  Every case ends with all ranks
agreeing on what happened; ``CASE_OK`` is printed by rank 0.
"""

import os
import sys
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from agentgarten_b200.infra.batch_transport import fetch_batch, prepare_batch  # noqa: E402
from agentgarten_b200.infra.model import ContextParallelContext  # noqa: E402


def _cp_context(size):
    from torch.distributed.device_mesh import init_device_mesh

    world = dist.get_world_size()
    if size == 1:
        return ContextParallelContext(None)
    mesh = init_device_mesh("cpu", (world // size, size), mesh_dim_names=("dp", "cp"))
    return ContextParallelContext(mesh["cp"])


def case_fetch_error_reaches_every_rank():
    """Rank 1's dataset raises: every rank gets a RuntimeError naming rank 1."""
    rank = dist.get_rank()
    context = ContextParallelContext(None)

    def batches():
        yield {"x": torch.full((2,), float(rank))}
        if rank == 1:
            raise ValueError("corrupt sample 17")
        yield {"x": torch.zeros(2)}

    iterator = batches()
    batch, exhausted, owner = fetch_batch(context, iterator, sequence_index=0)
    assert not exhausted and owner is None and float(batch["x"][0]) == rank
    try:
        fetch_batch(context, iterator, sequence_index=1)
    except RuntimeError as error:
        assert "rank 1" in str(error) and "corrupt sample 17" in str(error), str(error)
    else:
        raise AssertionError("the failure of rank 1 did not surface on rank %d" % rank)


def case_kernel_status_of_one_rank_stops_every_rank():
    """Rank 1 reports a timed-out peer wait (set on the host): the non-finite consensus of the
    next update raises KernelStatusError on every rank, naming the code, and so does a
    checkpoint save; after the word is cleared both proceed."""
    from agentgarten_b200.infra.nonfinite import synchronize_found_nonfinite
    from agentgarten_b200.ops import kernel_status

    rank = dist.get_rank()
    weight = torch.nn.Parameter(torch.ones(4))
    weight.grad = torch.ones(4)
    optimizer = torch.optim.SGD([weight], lr=0.1)
    scaler = torch.amp.GradScaler(device="cpu", enabled=False)
    assert synchronize_found_nonfinite(scaler, (optimizer,), fallback_device="cpu") is False
    kernel_status.inject(5 if rank == 1 else 0)
    try:
        synchronize_found_nonfinite(scaler, (optimizer,), fallback_device="cpu")
    except kernel_status.KernelStatusError as error:
        assert error.code == 5 and "kTimeoutPeer" in str(error), str(error)
    else:
        raise AssertionError("rank %d trained on after a peer timeout on rank 1" % rank)
    try:
        kernel_status.raise_for_status(kernel_status.read("cpu"), "checkpoint save")
    except kernel_status.KernelStatusError as error:
        assert "checkpoint save" in str(error)
    else:
        raise AssertionError("rank %d would have written a checkpoint" % rank)
    kernel_status.inject(None)
    assert kernel_status.read("cpu") == 0
    assert synchronize_found_nonfinite(scaler, (optimizer,), fallback_device="cpu") is False


def case_a_rank_that_leaves_ends_the_next_collective_of_the_others():
    """The last rank stops taking part between two steps (it simply never makes the next call):
    with the short process-group timeout of the run the others get an error from their next
    batch agreement instead of waiting for ever."""
    import time

    rank, world = dist.get_rank(), dist.get_world_size()   # the group was made with GROUP_TIMEOUT
    context = ContextParallelContext(None)
    iterator = iter([{"i": 0}] * 4)
    batch, exhausted, _ = fetch_batch(context, iterator, sequence_index=0)   # a step everyone takes
    assert not exhausted and batch == {"i": 0}
    began = time.monotonic()
    if rank == world - 1:
        time.sleep(8.0)                  # between steps: no collective of this rank is in flight
    else:
        try:
            fetch_batch(context, iterator, sequence_index=1)
        except RuntimeError as error:
            waited = time.monotonic() - began
            assert waited < 30.0, waited
            assert str(error), "the error carries the backend's message"
        else:
            raise AssertionError("rank %d went on without rank %d" % (rank, world - 1))
    # The group is broken now and cannot serve the worker's closing barrier: every rank waits
    # until all are past the timeout and ends here.
    time.sleep(max(0.0, 12.0 - (time.monotonic() - began)))
    if rank == 0:
        print("CASE_OK", sys.argv[1], flush=True)
    sys.stdout.flush()
    os._exit(0)


def case_uneven_end_stops_everyone():
    """Rank 0 runs out of data one batch early: all ranks report exhaustion together."""
    rank = dist.get_rank()
    context = ContextParallelContext(None)
    iterator = iter([{"i": 0}] * (2 if rank == 0 else 3))
    seen = 0
    while True:
        batch, exhausted, _ = fetch_batch(context, iterator, sequence_index=seen)
        if exhausted:
            break
        seen += 1
    assert seen == 2, seen


def case_cp_transport_shares_batch_and_rng():
    """Owner i % cp reads and prepares; the others receive tensors, structure and RNG state."""
    rank = dist.get_rank()
    context = _cp_context(2)
    assert context.enabled and context.size == 2

    def batches():
        for i in range(4):
            g = torch.Generator().manual_seed(1000 * rank + i)
            shared = torch.randn(3, 5, generator=g)
            yield {"latent": shared, "alias": shared, "ids": torch.arange(4) + 10 * rank + i,
                   "meta": {"caption": f"clip {rank}-{i}", "fps": 16.0}, "empty": torch.zeros(0, 2)}

    iterator = batches()
    for index in range(4):
        batch, exhausted, owner = fetch_batch(context, iterator, sequence_index=index)
        assert not exhausted and owner == index % 2
        assert (batch is not None) == (context.rank == owner)

        def prepare(b):
            torch.manual_seed(7 + index)  # the owner's generator state travels with the batch
            return {**b, "latent": b["latent"].double() * 2}

        out = prepare_batch(context, batch, owner_rank=owner, prepare=prepare)
        assert out["latent"].dtype == torch.float64 and out["alias"] is not None
        assert out["meta"]["caption"].startswith("clip ") and out["empty"].shape == (0, 2)
        gathered = [None] * 2
        dist.all_gather_object(gathered, (out["latent"].sum().item(), out["ids"].tolist(),
                                          out["meta"]["caption"], torch.rand(1).item()),
                               group=context.group)
        assert gathered[0] == gathered[1], gathered  # same data and same next random number
        owner_global = context.global_rank(owner)
        assert out["meta"]["caption"].startswith(f"clip {owner_global}-")


def case_cp_prepare_error_reaches_the_group():
    context = _cp_context(2)

    def prepare(b):
        raise FloatingPointError("encoder overflow")

    batch = {"x": torch.ones(2)} if context.rank == 0 else None
    try:
        prepare_batch(context, batch, owner_rank=0, prepare=prepare)
    except RuntimeError as error:
        assert "encoder overflow" in str(error)
    else:
        raise AssertionError("prepare failure did not surface")
    # an unpicklable leaf is reported the same way instead of hanging the receivers
    bad = {"x": torch.ones(2), "fn": (lambda: 0)} if context.rank == 0 else None
    try:
        prepare_batch(context, bad, owner_rank=0, prepare=lambda b: b)
    except RuntimeError as error:
        assert "prepare failed" in str(error)
    else:
        raise AssertionError("unpicklable batch did not surface")


def case_context_parallel_matches_single_group():
    """Two CP ranks reproduce the loss and gradients of the unsharded model on the same clip."""
    from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network

    from agentgarten_b200.models.diffusion import DiffusionModel
    from agentgarten_b200.parallel.engine import ParallelConfig

    config = tiny_config()
    losses, grads = {}, {}
    for cp in (1, 2):
        net = tiny_network(config, seed=0)
        cond = tiny_conditioner(config, seed=1)
        parallel = ParallelConfig(parameter_dtype="float32", context_parallel_size=cp,
                                  activation_checkpointing="none")
        model = DiffusionModel(net=net, conditioner=cond, text_dropout=0.0, parallel=parallel,
                               conditioner_parallel=ParallelConfig(parameter_dtype="float32",
                                                                   activation_checkpointing="none"))
        model.parallelize(torch.device("cpu"))
        batch = model.prepare_data_batch(synthetic_batch(frames=5, seed=3))
        torch.manual_seed(11)
        model.train()
        loss = None
        for _name, closure, _last in model.training_step_closures(batch, iteration=0):
            outputs, loss = closure()
            loss.backward()
        losses[cp] = float(loss)
        grads[cp] = {n: p.grad.clone() for n, p in model.net.named_parameters() if p.grad is not None}
    assert abs(losses[1] - losses[2]) < 1e-5 * max(1.0, abs(losses[1])), losses
    world = 2
    for name, full in grads[1].items():
        part = grads[2][name].clone()
        dist.all_reduce(part)  # each CP rank holds the gradient of its token shard
        scale = float(full.abs().max()) + 1e-8
        assert float((part - full).abs().max()) / scale < 2e-4 or \
            float((part / world - full).abs().max()) / scale < 2e-4, name


def case_node_groups_for_hybrid_sharding():
    """Four ranks as two nodes of two: shards are node-local, replicas pair equal local indices."""
    from agentgarten_b200.parallel.zero import node_groups

    rank = dist.get_rank()
    shard, replica = node_groups(2)
    assert dist.get_process_group_ranks(shard) == [rank - rank % 2, rank - rank % 2 + 1]
    assert dist.get_process_group_ranks(replica) == [rank % 2, rank % 2 + 2]
    value = torch.tensor([float(rank)])
    dist.all_reduce(value, group=replica)
    assert float(value) == 2 * (rank % 2) + 2
    assert node_groups(2) == (shard, replica)  # cached: groups are created once
    try:
        node_groups(3)
    except ValueError:
        pass
    else:
        raise AssertionError("4 ranks cannot form nodes of 3")


CASES = {name[5:]: fn for name, fn in list(globals().items()) if name.startswith("case_")}
# seconds after which a collective of the job's group gives up (the run's
# ``runtime.process_group_timeout_seconds``); cases that let one run out choose a short one
GROUP_TIMEOUT = {"a_rank_that_leaves_ends_the_next_collective_of_the_others": 4}


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo", timeout=timedelta(seconds=GROUP_TIMEOUT.get(sys.argv[1], 120)))
    try:
        CASES[sys.argv[1]]()
        dist.barrier()
        if dist.get_rank() == 0:
            print("CASE_OK", sys.argv[1])
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
