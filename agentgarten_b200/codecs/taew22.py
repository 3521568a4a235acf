"""Light "Super" decoder for normalised Wan 2.2 latents (encoding stays with the native VAE).

Parity: reference ``wm/codecs/taew22.py:14-88``.
"""

from __future__ import annotations

from pathlib import Path

import torch

from agentgarten_b200.codecs._taehv.taehv import TAEHV, StreamingTAEHV

__all__ = ["TAEW22SuperDecoder", "TAEW22SuperStream"]

_ARCH = "taew2_2_super"


def _check(latent: torch.Tensor) -> None:
    if not latent.is_floating_point():
        raise TypeError("Super decoder requires floating-point latents")
    if latent.ndim != 5 or latent.shape[1] != 48 or min(latent.shape) < 1:
        raise ValueError("Super decoder expects nonempty N,48,T,H,W latents")


class TAEW22SuperDecoder:
    """Decode diffusion-normalised latents to RGB in [-1,1].

    On CUDA the network runs in FP16 (its published inference recipe), on CPU in FP32.
    ``frames_per_pass`` latent frames advance together; memory is bounded by that chunk,
    not by the clip length, and the output does not depend on it.
    """

    def __init__(self, pretrained_path: str | Path | None, *, frames_per_pass: int = 4) -> None:
        self.pretrained_path = None if pretrained_path is None else str(pretrained_path)
        self.frames_per_pass = max(1, int(frames_per_pass))
        self._model: TAEHV | None = None

    def _get_model(self, device: torch.device) -> TAEHV:
        if self._model is None:
            self._model = TAEHV(self.pretrained_path, arch_name=_ARCH).eval().requires_grad_(False)
        dtype = torch.float16 if device.type == "cuda" else torch.float32
        self._model = self._model.to(device=device, dtype=dtype)
        if device.type == "cuda":
            self._model = self._model.to(memory_format=torch.channels_last)
        return self._model

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        """``[N,48,T,H,W] -> [N,3,4T-3,16H,16W]``, in the dtype of ``latent``."""
        _check(latent)
        stream = self.stream(latent.device)
        pieces = [stream.decode(latent[:, :, start:start + self.frames_per_pass])
                  for start in range(0, latent.shape[2], self.frames_per_pass)]
        return torch.cat(pieces, dim=2)

    def stream(self, device: str | torch.device) -> "TAEW22SuperStream":
        """Independent recurrence on the shared frozen weights."""
        return TAEW22SuperStream(self._get_model(torch.device(device)))


class TAEW22SuperStream:
    """Decode contiguous latent chunks; the three start-up frames are trimmed once."""

    def __init__(self, model: TAEHV) -> None:
        self._stream = StreamingTAEHV(model)
        self._shape: tuple[int, int, int] | None = None

    def reset(self) -> None:
        self._stream.reset()
        self._shape = None

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        """The first chunk of ``T`` latent frames yields ``4T-3`` RGB frames, later ones ``4T``."""
        _check(latent)
        weight = next(self._stream.taehv.parameters())
        if latent.device != weight.device:
            raise ValueError("stream latent device must match decoder device")
        shape = (latent.shape[0], latent.shape[3], latent.shape[4])
        if self._shape is not None and shape != self._shape:
            raise ValueError("reset the stream before changing batch or spatial shape")
        self._shape = shape
        with torch.autocast(device_type=latent.device.type, enabled=False):
            # The tiny decoder consumes normalised latents directly: no mean/std here.
            video = self._stream.decode_chunk(latent.transpose(1, 2).to(weight.dtype))
            return (video.transpose(1, 2) * 2 - 1).to(latent.dtype)
