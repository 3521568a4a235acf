"""agentgarten_b200: a Blackwell-native (sm_100a) training and streaming-inference
framework for geometry-conditioned video world models.

The package provides a Cosmos3-Nano-shaped DiT conditioned on depth/normal latents,
three training recipes (bidirectional rectified flow, block-causal autoregression with
teacher or diffusion forcing, Adversarial-Forcing distillation with exact R1/R2) and a
block-by-block KV-cache streaming sampler.  PyTorch is the framework layer; the hot
operators live in ``agentgarten_b200/csrc`` as hand-written CUDA kernels (tcgen05 /
TMEM tensor-core tiles fed by TMA, peer-memory collectives over NVLink).

The historical import root ``wm`` is kept as an alias package so that configuration
targets such as ``wm.models.diffusion.DiffusionModel`` keep resolving.
"""

from .__about__ import __version__

__all__ = ["__version__"]
