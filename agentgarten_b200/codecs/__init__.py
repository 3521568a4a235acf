"""Latent video codecs: the Wan 2.2 VAE and its light "Super" decoder.

Parity: reference ``wm/codecs/__init__.py:1-6``.
"""

from agentgarten_b200.codecs.taew22 import TAEW22SuperDecoder, TAEW22SuperStream
from agentgarten_b200.codecs.wan22 import Wan22Stream, Wan22VAECodec

__all__ = ["TAEW22SuperDecoder", "TAEW22SuperStream", "Wan22Stream", "Wan22VAECodec"]
