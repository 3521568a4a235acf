"""DMD-GAN with exact R1/R2 (weight 0.075 = 30 * 0.05^2, the local scale of the
finite-difference recipe); the teacher runs un-traced because it is differentiated in
forward mode."""

from agentgarten_b200.configs.experiments.cosmos3 import parallel
from agentgarten_b200.configs.experiments.cosmos3.dmd_gan import build_config as dmd_gan_config
from agentgarten_b200.infra.config import LazyDict


def build_config() -> LazyDict:
    config = dmd_gan_config()
    config.job.output_dir = "${paths.output_root}/cosmos3/dmd_gan_exact"
    config.model.gan.regularization = "exact"
    config.model.gan.exact_regularization_weight = 0.075
    config.model.real_score_parallel = parallel(activation_checkpointing="full", compile=False)
    return config
