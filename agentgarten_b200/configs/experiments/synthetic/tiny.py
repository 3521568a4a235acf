"""A two-layer Cosmos3-shaped model on synthetic cached latents.

``python -m agentgarten_b200.train experiment=synthetic/tiny job.output_dir=/tmp/run
runtime.device=cpu runtime.backend=gloo`` exercises the whole training path (configuration,
model placement, optimizer engine, loader, callbacks, checkpoints) in seconds on any
machine; on a GPU box the same recipe runs the native kernels (widths are multiples of the
tile sizes they need).
"""

import torch

from agentgarten_b200.configs.base import make_base_config
from agentgarten_b200.configs.experiments.cosmos3 import optimizer, parallel
from agentgarten_b200.data.loader import StatefulDataLoader
from agentgarten_b200.data.video import SyntheticLatentDataset
from agentgarten_b200.infra.config import LazyCall, LazyDict
from agentgarten_b200.infra.optim import LinearWarmup
from agentgarten_b200.models.diffusion import DiffusionModel
from agentgarten_b200.models.flow import RectifiedFlowSchedule
from agentgarten_b200.networks.cosmos3 import Cosmos3Config, build_network
from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner

VOCAB = 512


def _loader(length: int, *, shuffle: bool) -> LazyDict:
    return LazyCall(StatefulDataLoader)(
        dataset=LazyCall(SyntheticLatentDataset)(
            length=length, latent_frames=3, latent_height=8, latent_width=8, text_tokens=12,
            vocab_size=VOCAB),
        batch_size=1, shuffle=shuffle, num_workers=0)


def build_config() -> LazyDict:
    config = make_base_config()
    config.cosmos3 = LazyCall(Cosmos3Config)(
        hidden_size=256, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=2,
        num_key_value_heads=1, head_dim=128, vocab_size=VOCAB, mrope_section=(24, 20, 20),
        text_bucket_tokens=16, special_tokens={"eos_token_id": 1, "start_of_generation": 2})
    config.model_parallel = {"fsdp_mesh_shape": None, "context_parallel_size": 1}
    config.model = LazyCall(DiffusionModel)(
        net=LazyCall(build_network)(config="${cosmos3}", init_device="meta", lora=None),
        conditioner=LazyCall(Cosmos3Conditioner)(config="${cosmos3}", codec=None, geometry_noise_sigma=0.0,
                                                empty_prompt_ids=[3, 4, 1]),
        schedule=LazyCall(RectifiedFlowSchedule)(shift=5.0, train_distribution="waver"),
        text_dropout=0.1, parallel=parallel(activation_checkpointing="none", random_init_seed=0),
        conditioner_parallel=parallel(activation_checkpointing="none", compile=False, random_init_seed=1),
        sampling={"num_steps": 4, "guidance": 1.0, "seed": 0})
    config.optimizer = optimizer(1e-3)
    config.scheduler = LazyCall(torch.optim.lr_scheduler.LambdaLR)(
        lr_lambda=LazyCall(LinearWarmup)(warmup_steps=2, start_factor=0.1))
    config.dataloader_train = _loader(64, shuffle=True)
    config.dataloader_val = _loader(4, shuffle=False)
    config.train.max_iterations = 6
    config.train.checkpoint_interval = 3
    config.train.validation_interval = 3
    config.train.max_val_steps = 2
    config.trainer.callbacks.metrics.every_n = 1
    return config
