"""Few-step distillation: student / frozen teacher / fake score; 5 fake-score updates per
student update; cadences count student updates."""

from agentgarten_b200.configs.experiments.cosmos3 import (conditioner, cosmos3_base,
                                                          gen_initialization, network, optimizer, parallel)
from agentgarten_b200.infra.config import LazyCall, LazyDict
from agentgarten_b200.models.dmd import DMDModel

SAMPLING = {"num_steps": 4, "seed": 2026}


def build_config() -> LazyDict:
    config = cosmos3_base(name="dmd", pixel_frames=81, sampling=dict(SAMPLING))
    config.model = LazyCall(DMDModel)(
        student=network(), real_score=network(), fake_score=network(), conditioner=conditioner(),
        block_frames=4, score_shift=5.0, real_score_guidance=6.0, fake_score_updates_per_student=5,
        dmd_loss_scale=0.5,
        student_parallel=parallel(activation_checkpointing="full", compile=False),
        score_parallel=parallel(activation_checkpointing="full"),
        conditioner_parallel=parallel(activation_checkpointing="none", compile=False),
        sampling=dict(SAMPLING))
    config.optimizer = {"student": optimizer(2e-6, betas=(0.0, 0.999)),
                        "fake_score": optimizer(4e-7, betas=(0.0, 0.999))}
    inits = config.train.model_initializations
    inits.student = gen_initialization("student")
    inits.real_score = gen_initialization("real_score", frozen=True)
    inits.fake_score = gen_initialization("fake_score")
    config.train.checkpoint_interval = 10
    config.train.validation_interval = 10
    config.trainer.grad_accum_steps = 2
    return config
