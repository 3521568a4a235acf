"""Worker of the checkpoint-interchange test (this package's side), two Gloo ranks on CPU.

``torchrun ... tests/interchange_worker.py <output> --directory D [--resume]`` does what
``baseline/reference_probe.py checkpoint`` does with the reference package: without
``--resume`` two optimizer updates, a checkpoint ``iter_000000002`` under ``D`` and a third
update; with it, a fresh job loads ``D/latest`` (written by either implementation) and runs
the third update.  Rank 0 writes the third update's loss (mean over ranks) to ``output``.
"""

import argparse
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("output")
    parser.add_argument("--directory", required=True)
    parser.add_argument("--resume", action="store_true")
    args = parser.parse_args()

    from reference_probe import batch_of, seeded_  # shared seeding of weights and batches

    from agentgarten_b200.infra import distributed
    from agentgarten_b200.infra.callbacks import CallbackGroup, GradClip
    from agentgarten_b200.infra.checkpoint import DistributedCheckpointer
    from agentgarten_b200.infra.config import LazyCall
    from agentgarten_b200.infra.optim import FusedAdam, LinearWarmup
    from agentgarten_b200.infra.trainer import Trainer
    from agentgarten_b200.models.diffusion import DiffusionModel
    from agentgarten_b200.networks.cosmos3 import Cosmos3Config, build_network
    from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
    from agentgarten_b200.parallel.engine import ParallelConfig

    torch.set_num_threads(2)
    device = distributed.init(device="cpu", backend="gloo")
    rank = distributed.get_rank()
    config = Cosmos3Config(hidden_size=256, intermediate_size=1024, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=128,
                           mrope_section=(12, 10, 10), text_bucket_tokens=16,
                           special_tokens={"eos_token_id": 1, "start_of_generation": 2})
    sharded = ParallelConfig(parameter_dtype="float32", fully_shard=True, activation_checkpointing="none",
                             compile=False)
    model = DiffusionModel(
        net=build_network(config, init_device="meta"),
        conditioner=Cosmos3Conditioner(config=config, codec=None, geometry_noise_sigma=0.0,
                                       init_device="meta", empty_prompt_ids=(3, 4, 5)),
        text_dropout=0.0, parallel=sharded, conditioner_parallel=sharded)
    model.parallelize(device)
    seeded_(model.net, 0 if not args.resume else 50)
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
    checkpointer = DistributedCheckpointer(args.directory, async_mode="disabled")

    def update(step: int) -> float:
        torch.manual_seed(1000 * step + rank)
        data = model.prepare_data_batch(batch_of(5, seed=100 * step + rank))
        result = trainer.training_step(model, scaler, data, iteration=step)
        loss = result.loss.detach().clone()
        dist.all_reduce(loss)
        return float(loss) / dist.get_world_size()

    if args.resume:
        loaded = checkpointer.load(model, model.optimizer_dict, model.scheduler_dict, scaler, path="latest")
        assert loaded.iteration == 2, loaded
    else:
        for step in range(2):
            update(step)
        checkpointer.save(model, model.optimizer_dict, model.scheduler_dict, scaler, iteration=2)
        checkpointer.finalize()
    loss = update(2)
    if rank == 0:
        torch.save({"loss": loss, "lr": optimizer.param_groups[0]["lr"]}, args.output)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
