"""Tiny recurrent video autoencoder (TAEHV family) on a chunked temporal pipeline.

Every block sees frames in causal order and needs at most one remembered frame (memory
blocks) or a short backlog (temporal pooling). So instead of choosing between "all
frames at once" and a frame-by-frame work queue, one routine pushes a *chunk* of frames
through the whole stack with a per-block state: a clip decoded in one chunk is the
parallel mode, chunks of one frame are the bounded-memory mode, and a live stream simply
keeps the state between calls. All three produce the same frames.

The module numbering follows the published ``taew2_2`` / ``*_super`` checkpoints so they
load without a key map.

Parity: reference ``wm/codecs/_taehv/taehv.py:14-464`` (blocks, architectures by
checkpoint name, ``encode_video`` / ``decode_video``, ``StreamingTAEHV``).
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.nn.functional as F
from torch import nn

from agentgarten_b200.ops.conv import conv_frames, depthwise_frames

__all__ = ["TAEHV", "StreamingTAEHV", "TemporalState", "run_stack"]

# name fragment -> (pixel patch, latent channels, encoder time halvings, decoder time doublings)
_ARCHITECTURES = {
    "taehv1_5": (2, 32, None, None),
    "taew2_2": (2, 48, None, None),
    "taeh3": (2, 24, None, None),
    "taeltx": (4, 128, (True, True, True), (True, True, True)),
}


class FrameConv(nn.Conv2d):
    """A frame convolution that runs in the tensor-core kernel when its input allows."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return conv_frames(self, x)


def _conv3(n_in: int, n_out: int, **kwargs) -> nn.Conv2d:
    return FrameConv(n_in, n_out, 3, padding=1, **kwargs)


class Clamp(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.tanh(x / 3) * 3


class MemBlock(nn.Module):
    """Three 3x3 convolutions over the current and the previous frame, plus a skip."""

    def __init__(self, n_in: int, n_out: int) -> None:
        super().__init__()
        self.conv = nn.Sequential(_conv3(n_in * 2, n_out), nn.ReLU(inplace=True), _conv3(n_out, n_out),
                                  nn.ReLU(inplace=True), _conv3(n_out, n_out))
        self.skip = nn.Conv2d(n_in, n_out, 1, bias=False) if n_in != n_out else nn.Identity()
        self.act = nn.ReLU(inplace=True)

    def forward(self, x: torch.Tensor, past: torch.Tensor) -> torch.Tensor:
        # Slots 1 and 3 of ``conv`` and ``act`` are the ReLUs applied inside the convolutions here.
        conv = self.conv
        skip = x if isinstance(self.skip, nn.Identity) else conv_frames(self.skip, x)
        h = conv_frames(conv[0], torch.cat([x, past], 1), relu=True)
        h = conv_frames(conv[2], h, relu=True)
        return conv_frames(conv[4], h, residual=skip, relu=True)


class SuperMemBlock(nn.Module):
    """ConvNeXt-style memory block of the larger decoder: 7x7 depthwise, 4x bottleneck."""

    def __init__(self, n_f: int) -> None:
        super().__init__()
        self.conv = nn.Sequential(
            nn.Conv2d(n_f * 2, n_f * 2, 7, padding=3, groups=n_f * 2, bias=False),
            nn.Conv2d(n_f * 2, n_f * 4, 1), nn.ReLU(inplace=True),
            nn.Conv2d(n_f * 4, n_f, 1, bias=False))

    def forward(self, x: torch.Tensor, past: torch.Tensor) -> torch.Tensor:
        conv = self.conv
        h = depthwise_frames(conv[0], torch.cat([x, past], 1))
        h = conv_frames(conv[1], h, relu=True)
        return conv_frames(conv[3], h, residual=x)


class TPool(nn.Module):
    """Merge ``stride`` consecutive frames into one with a 1x1 convolution."""

    def __init__(self, n_f: int, stride: int) -> None:
        super().__init__()
        self.stride = stride
        self.conv = nn.Conv2d(n_f * stride, n_f, 1, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _, c, h, w = x.shape
        return conv_frames(self.conv, x.reshape(-1, self.stride * c, h, w))


class TGrow(nn.Module):
    """Split one frame into ``stride`` consecutive frames with a 1x1 convolution."""

    def __init__(self, n_f: int, stride: int) -> None:
        super().__init__()
        self.stride = stride
        self.conv = nn.Conv2d(n_f, n_f * stride, 1, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _, c, h, w = x.shape
        return conv_frames(self.conv, x).reshape(-1, c, h, w)


class TemporalState:
    """What a stack remembers between chunks: one slot per block."""

    def __init__(self, blocks: int) -> None:
        self.slots: list[torch.Tensor | None] = [None] * blocks

    def reset(self) -> None:
        self.slots = [None] * len(self.slots)


def run_stack(stack: Sequence[nn.Module], frames: torch.Tensor, state: TemporalState | None = None) -> torch.Tensor | None:
    """Advance ``stack`` by a chunk ``[N,T,C,H,W]``; returns ``[N,T',C',H',W']`` or ``None``.

    ``None`` means the chunk ended inside a pooling block's backlog and no frame came out.
    Without ``state`` the chunk is treated as a complete clip that starts from empty memory.
    """
    if frames.ndim != 5:
        raise ValueError(f"expected [N,T,C,H,W] frames, got {tuple(frames.shape)}")
    state = state or TemporalState(len(stack))
    n = frames.shape[0]
    x = frames
    for index, block in enumerate(stack):
        t = x.shape[1]
        if isinstance(block, (MemBlock, SuperMemBlock)):
            before = state.slots[index]
            if before is None:
                before = torch.zeros_like(x[:, :1])
            past = torch.cat([before, x[:, :-1]], dim=1) if t > 1 else before
            state.slots[index] = x[:, -1:].clone()
            x = block(x.flatten(0, 1), past.flatten(0, 1)).unflatten(0, (n, t))
        elif isinstance(block, TPool):
            if block.stride > 1:
                backlog = state.slots[index]
                if backlog is not None:
                    x = torch.cat([backlog, x], dim=1)
                whole = (x.shape[1] // block.stride) * block.stride
                state.slots[index] = x[:, whole:].clone() if whole < x.shape[1] else None
                if whole == 0:
                    return None
                x = x[:, :whole]
            x = block(x.flatten(0, 1)).unflatten(0, (n, x.shape[1] // block.stride))
        elif isinstance(block, TGrow):
            x = block(x.flatten(0, 1)).unflatten(0, (n, t * block.stride))
        else:
            x = block(x.flatten(0, 1)).unflatten(0, (n, t))
    return x


def _stage(kind: str, width: int) -> list[nn.Module]:
    block = SuperMemBlock if kind == "super" else (lambda n: MemBlock(n, n))
    return [block(width) for _ in range(3)]


class TAEHV(nn.Module):
    """Encoder and decoder of the tiny autoencoder; the architecture follows the checkpoint name.

    ``arch_name`` (or, when absent, ``checkpoint_path``) selects patch size and latent
    channels by the fragments ``taew2_2`` / ``taehv1_5`` / ``taeh3`` / ``taeltx``; a
    ``_super`` suffix selects the wider decoder. ``checkpoint_path=None`` leaves the
    weights at their initial values. The chunk-grouping quirks of the ``taeh3`` and
    ``taecvx`` variants of the original project are not implemented.
    """

    def __init__(self, checkpoint_path: str | None = "taehv.pth", encoder_time_downscale=None,
                 decoder_time_upscale=None, decoder_space_upscale=None, patch_size: int | None = None,
                 latent_channels: int | None = None, arch_name: str | None = None) -> None:
        super().__init__()
        self.arch_name = str(arch_name or checkpoint_path or "")
        for fragment, (patch, channels, down, up) in _ARCHITECTURES.items():
            if fragment in self.arch_name:
                patch_size, latent_channels = patch_size or patch, latent_channels or channels
                encoder_time_downscale = encoder_time_downscale or down
                decoder_time_upscale = decoder_time_upscale or up
        self.patch_size = patch_size or 1
        self.latent_channels = latent_channels or 16
        self.image_channels = 3
        t_down = tuple(encoder_time_downscale or (True, True, False))
        t_up = tuple(decoder_time_upscale or (False, True, True))
        s_up = tuple(decoder_space_upscale or (True, True, True))
        if len(t_up) == 2:
            t_up = (False, *t_up)
        pixels = self.image_channels * self.patch_size ** 2

        encoder: list[nn.Module] = [_conv3(pixels, 64), nn.ReLU(inplace=True)]
        for halve in t_down:
            encoder += [TPool(64, 2 if halve else 1), _conv3(64, 64, stride=2, bias=False), *_stage("plain", 64)]
        encoder.append(_conv3(64, self.latent_channels))
        self.encoder = nn.Sequential(*encoder)

        decoder: list[nn.Module]
        if "_super" in self.arch_name:
            widths = (512, 256, 128, 64)
            decoder = [FrameConv(self.latent_channels, widths[0], 1, bias=False)]
            for level in range(3):
                grow = 2 if s_up[level] else 1
                decoder += [*_stage("super", widths[level]),
                            _conv3(widths[level], widths[level + 1] * grow * grow), nn.ReLU(inplace=True),
                            nn.PixelShuffle(grow), TGrow(widths[level + 1], 2 if t_up[level] else 1)]
            decoder.append(_conv3(widths[3], pixels))
        else:
            widths = (256, 128, 64, 64)
            decoder = [Clamp(), _conv3(self.latent_channels, widths[0]), nn.ReLU(inplace=True)]
            for level in range(3):
                decoder += [*_stage("plain", widths[level]), nn.Upsample(scale_factor=2 if s_up[level] else 1),
                            TGrow(widths[level], 2 if t_up[level] else 1),
                            _conv3(widths[level], widths[level + 1], bias=False)]
            decoder += [nn.ReLU(inplace=True), _conv3(widths[3], pixels)]
        self.decoder = nn.Sequential(*decoder)

        self.t_downscale = 2 ** sum(b.stride == 2 for b in self.encoder if isinstance(b, TPool))
        self.t_upscale = 2 ** sum(b.stride == 2 for b in self.decoder if isinstance(b, TGrow))
        self.frames_to_trim = self.t_upscale - 1
        if checkpoint_path is not None:
            self.load_state_dict(self._fit_time_growth(_read_weights(str(checkpoint_path))))

    def _fit_time_growth(self, weights: dict) -> dict:
        """Checkpoints carry 2x temporal growth everywhere; keep the last-frame half where it is off."""
        own = self.state_dict()
        for index, block in enumerate(self.decoder):
            key = f"decoder.{index}.conv.weight"
            if isinstance(block, TGrow) and weights[key].shape[0] > own[key].shape[0]:
                weights[key] = weights[key][-own[key].shape[0]:]
        return weights

    # ---- pixel <-> patch helpers ---------------------------------------------------------
    def preprocess_input_frames(self, x: torch.Tensor) -> torch.Tensor:
        return F.pixel_unshuffle(x, self.patch_size) if self.patch_size > 1 else x

    def postprocess_output_frames(self, x: torch.Tensor) -> torch.Tensor:
        if self.patch_size > 1:
            x = F.pixel_shuffle(x, self.patch_size)
        return x.clamp_(0, 1)

    # ---- whole clips -------------------------------------------------------------------------
    def _run_clip(self, stack: nn.Sequential, x: torch.Tensor, parallel: bool) -> torch.Tensor:
        if parallel:
            return run_stack(stack, x)
        state = TemporalState(len(stack))
        pieces = [run_stack(stack, x[:, t:t + 1], state) for t in range(x.shape[1])]
        return torch.cat([p for p in pieces if p is not None], dim=1)

    def encode_video(self, x: torch.Tensor, parallel: bool = True, show_progress_bar: bool = False) -> torch.Tensor:
        """``[N,T,3,H,W]`` RGB in [0,1] to ``[N,T/t_downscale,C,H/8p,W/8p]`` latents."""
        x = self.preprocess_input_frames(x)
        short = -x.shape[1] % self.t_downscale
        if short:  # repeat the last frame to a whole pooling group
            x = torch.cat([x, x[:, -1:].expand(-1, short, -1, -1, -1)], dim=1)
        return self._run_clip(self.encoder, x, parallel)

    def decode_video(self, x: torch.Tensor, parallel: bool = True, show_progress_bar: bool = False) -> torch.Tensor:
        """``[N,T,C,h,w]`` latents to ``[N,T*t_upscale-(t_upscale-1),3,H,W]`` RGB in [0,1]."""
        frames = self.postprocess_output_frames(self._run_clip(self.decoder, x, parallel))
        return frames[:, self.frames_to_trim:]


def _read_weights(path: str) -> dict:
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file
        return load_file(path)
    return torch.load(path, map_location="cpu", weights_only=True)


class StreamingTAEHV(nn.Module):
    """Live wrapper: feed frames or latents as they arrive, collect outputs as they are due.

    ``encode`` returns the latents a chunk of pixel frames completes (``None`` while a
    pooling group is still open); ``flush_encoder`` repeats the last frame to close it.
    ``decode`` returns all frames a chunk of latents produces, minus the start-up frames
    that align the decoder with the reference VAE, which are dropped once per stream.
    """

    def __init__(self, taehv: TAEHV) -> None:
        super().__init__()
        self.taehv = taehv
        self.reset()

    def reset(self) -> None:
        self.encoder_state = TemporalState(len(self.taehv.encoder))
        self.decoder_state = TemporalState(len(self.taehv.decoder))
        self.n_frames_encoded = 0
        self.n_frames_decoded = 0
        self._pending: list[torch.Tensor] = []
        self._last_input: torch.Tensor | None = None

    def encode(self, x: torch.Tensor) -> torch.Tensor | None:
        if x.ndim != 5 or x.shape[2] != self.taehv.image_channels:
            raise ValueError(f"expected [N,T,3,H,W] frames, got {tuple(x.shape)}")
        self._last_input = x[:, -1:]
        self.n_frames_encoded += x.shape[1]
        return run_stack(self.taehv.encoder, self.taehv.preprocess_input_frames(x), self.encoder_state)

    def flush_encoder(self) -> list[torch.Tensor]:
        short = -self.n_frames_encoded % self.taehv.t_downscale
        if self._last_input is None or not short:
            return []
        latent = self.encode(self._last_input.expand(-1, short, -1, -1, -1))
        return [] if latent is None else list(latent.split(1, dim=1))

    def decode(self, x: torch.Tensor | None = None) -> torch.Tensor | None:
        """With a latent chunk: decode it and return its first due frame; without: the next one."""
        if x is not None:
            if x.ndim != 5 or x.shape[2] != self.taehv.latent_channels:
                raise ValueError(f"expected [N,T,{self.taehv.latent_channels},h,w] latents, got {tuple(x.shape)}")
            raw = run_stack(self.taehv.decoder, x, self.decoder_state)
            skip = max(0, self.taehv.frames_to_trim - self.n_frames_decoded)
            self.n_frames_decoded += raw.shape[1]
            frames = self.taehv.postprocess_output_frames(raw[:, skip:])
            self._pending.extend(frames.split(1, dim=1))
        return self._pending.pop(0) if self._pending else None

    def decode_chunk(self, x: torch.Tensor) -> torch.Tensor:
        """All frames a latent chunk produces, as one tensor (empty queue required)."""
        first = self.decode(x)
        return torch.cat([first, *self.flush_decoder()], dim=1)

    def flush_decoder(self) -> list[torch.Tensor]:
        frames, self._pending = self._pending, []
        return frames

    def flush(self) -> list[torch.Tensor]:
        frames = []
        for latent in self.flush_encoder():
            first = self.decode(latent)
            if first is not None:
                frames.append(first)
            frames.extend(self.flush_decoder())
        frames.extend(self.flush_decoder())
        return frames
