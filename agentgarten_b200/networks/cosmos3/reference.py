"""Training-free conditioning of a streamed block on clean reference images.

The reference latents are embedded as clean tokens (no timestep embedding and no
first-frame marker) at time slots just *before* the stream's first frame, with their own
unscaled patch-grid coordinates, and are run through the layer stack together with the
noisy block. Every query of that group reads the prompt, the committed history and the
whole group; nothing about the references is written to the cache, so the following
``commit`` and later blocks are untouched. Without references the call is exactly
``stream.denoise``.

Parity: reference ``wm/networks/cosmos3/reference.py:24-118``.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch

from agentgarten_b200 import ops

from .network import Cosmos3Condition, rgb_tokens
from .streaming import Cosmos3Stream

__all__ = ["denoise_with_references"]


def _reference_positions(height: int, width: int, time: torch.Tensor) -> torch.Tensor:
    """``[B, h*w, 3]`` (time, row, column) with integer patch coordinates."""
    rows = torch.arange(height, device=time.device, dtype=torch.float32)
    cols = torch.arange(width, device=time.device, dtype=torch.float32)
    out = torch.empty(time.shape[0], height, width, 3, device=time.device, dtype=torch.float32)
    out[..., 0] = time[:, None, None]
    out[..., 1] = rows[None, :, None]
    out[..., 2] = cols[None, None, :]
    return out.flatten(1, 2)


@torch.inference_mode()
def denoise_with_references(stream: Cosmos3Stream, noisy: torch.Tensor, sigma: torch.Tensor,
                            condition: Cosmos3Condition,
                            references: Sequence[torch.Tensor]) -> torch.Tensor:
    """Velocity of the noisy block given ``references`` (each ``[1, C, 1, H, W]``, clean)."""
    if not references:
        return stream.denoise(noisy, sigma, condition)
    stream.validate_chunk(noisy, condition)
    network = stream.network
    if network.context_parallel is not None:
        raise ValueError("reference queries do not support context parallelism")
    if len(stream.layers) != len(network.layers):
        raise RuntimeError("Prefill C0 before using reference images")
    config = network.config

    tokens, positions = stream.embed_chunk(noisy, sigma, condition)
    origin = condition.text.valid_lengths.to(tokens.device, torch.float32) + config.temporal_modality_margin
    pieces, places = [], []
    for index, image in enumerate(references):
        if (image.ndim != 5 or tuple(image.shape[:3]) != (1, config.latent_channels, 1)
                or image.device != noisy.device):
            raise ValueError("Reference must be a single clean image latent on the query device")
        # sigma None: a clean image gets no timestep embedding; reference=False: the learned
        # marker belongs to the stream's own first frame only.
        pieces.append(network.embed_rgb(image, None, reference=False, condition=condition).flatten(1, 2))
        places.append(_reference_positions(image.shape[-2] // config.patch_size,
                                           image.shape[-1] // config.patch_size,
                                           origin + index - len(references)))
    extra = sum(piece.shape[1] for piece in pieces)

    def attend(index, queries, keys, values):
        cache = stream.layers[index]
        end = cache.text_tokens + cache.frames * cache.frame_tokens
        key = torch.cat((cache.key[:, :end], keys[0]), dim=1)
        value = torch.cat((cache.value[:, :end], values[0]), dim=1)
        return [ops.attention(queries[0], key, value, None)]

    (hidden,), _ = network.run_layers([torch.cat((*pieces, tokens), dim=1)],
                                      [torch.cat((*places, positions), dim=1)], attend)
    return network.decode_velocity(rgb_tokens(hidden[:, extra:], noisy.shape[2], stream.grid), stream.grid)
