"""Bidirectional rectified flow: lr 3e-5, accumulation 4, 81 pixel frames, 35 sampling steps."""

from agentgarten_b200.configs.experiments.cosmos3 import (conditioner, cosmos3_base,
                                                          gen_initialization, network, optimizer, parallel)
from agentgarten_b200.infra.config import LazyCall, LazyDict
from agentgarten_b200.models.diffusion import DiffusionModel
from agentgarten_b200.models.flow import RectifiedFlowSchedule

SAMPLING = {"num_steps": 35, "guidance": 6.0, "seed": 2026}


def build_config() -> LazyDict:
    config = cosmos3_base(name="bidirectional", pixel_frames=81, sampling=dict(SAMPLING))
    config.model = LazyCall(DiffusionModel)(
        net=network(), conditioner=conditioner(),
        schedule=LazyCall(RectifiedFlowSchedule)(shift=5.0, train_distribution="waver"),
        text_dropout=0.1, parallel=parallel(),
        conditioner_parallel=parallel(activation_checkpointing="none", compile=False),
        sampling=dict(SAMPLING))
    config.optimizer = optimizer(3e-5)
    config.train.model_initializations.net = gen_initialization("net")
    config.trainer.grad_accum_steps = 4
    return config
