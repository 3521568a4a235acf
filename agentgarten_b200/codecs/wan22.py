"""Wan 2.2 video VAE: 16x spatial / 4x temporal compression into 48 latent channels.

The module tree keeps the parameter names of the released ``Wan2.2_VAE.pth`` checkpoint so
that it loads without a key map; everything around the weights is organised for a large
single GPU:

* the recurrence of the causal convolutions lives in an explicit :class:`CausalState`
  (one per stream) instead of positional cache lists, so one set of frozen weights can
  serve any number of concurrent encode/decode streams;
* convolutions pad space inside the convolution and only concatenate the (at most two)
  remembered frames in time, so no padded copy of a full-resolution activation is made;
* after the first latent frame the decoder advances several latent frames per pass
  (bit-for-bit the same recurrence as one frame at a time, with far fewer launches);
* on CUDA the activations run channels-last in bf16, which is the layout the tensor-core
  convolution kernels want.

Parity: reference ``wm/codecs/wan22.py:29-1135`` (layers, chunked causal encode, frame by
frame decode, latent normalisation tables, ``Wan22VAECodec`` surface).
"""

from __future__ import annotations

import math
from pathlib import Path
from typing import Sequence

import torch
import torch.nn.functional as F
from torch import nn

from agentgarten_b200.ops.conv import conv_frames, conv_volume, conv_volume_causal, eligible
from agentgarten_b200.utils import log
from agentgarten_b200.utils.misc import prefetch

__all__ = ["CausalState", "Wan22VAE", "Wan22VAECodec", "Wan22Stream", "LATENT_MEAN", "LATENT_STD",
           "pixel_fold", "pixel_unfold", "to_channels_last"]

# Per-channel statistics of the released 48-channel latent space.
LATENT_MEAN = (
    -0.2289, -0.0052, -0.1323, -0.2339, -0.2799, 0.0174, 0.1838, 0.1557, -0.1382, 0.0542, 0.2813,
    0.0891, 0.1570, -0.0098, 0.0375, -0.1825, -0.2246, -0.1207, -0.0698, 0.5109, 0.2665, -0.2108,
    -0.2158, 0.2502, -0.2055, -0.0322, 0.1109, 0.1567, -0.0729, 0.0899, -0.2799, -0.1230, -0.0313,
    -0.1649, 0.0117, 0.0723, -0.2839, -0.2083, -0.0520, 0.3748, 0.0152, 0.1957, 0.1433, -0.2944,
    0.3573, -0.0548, -0.1681, -0.0667)
LATENT_STD = (
    0.4765, 1.0364, 0.4514, 1.1677, 0.5313, 0.4990, 0.4818, 0.5013, 0.8158, 1.0344, 0.5894, 1.0901,
    0.6885, 0.6165, 0.8454, 0.4978, 0.5759, 0.3523, 0.7135, 0.6804, 0.5833, 1.4146, 0.8986, 0.5659,
    0.7069, 0.5338, 0.4889, 0.4917, 0.4069, 0.4999, 0.6866, 0.4093, 0.5709, 0.6065, 0.6415, 0.4944,
    0.5726, 1.2042, 0.5458, 1.6887, 0.3971, 1.0600, 0.3943, 0.5537, 0.5444, 0.4089, 0.7468, 0.7744)
# the names the reference module gives the same tables
WAN22_LATENTS_MEAN, WAN22_LATENTS_STD = LATENT_MEAN, LATENT_STD

_HISTORY = 2  # frames of left context a temporal kernel of three needs


class CausalState:
    """Recurrent memory of one encode or decode stream.

    ``history`` maps a module to the trailing frames of its previous inputs. ``chunks``
    counts the chunks already consumed: the very first chunk is special in three places
    (temporal up-sampling is skipped, the duplicated shortcut is trimmed, and temporal
    down-sampling only records its input).
    """

    def __init__(self) -> None:
        self.history: dict[nn.Module, torch.Tensor] = {}
        self.chunks = 0

    @property
    def first(self) -> bool:
        return self.chunks == 0

    def advance(self) -> None:
        self.chunks += 1

    def reset(self) -> None:
        self.history.clear()
        self.chunks = 0


def pixel_fold(x: torch.Tensor, patch: int = 2) -> torch.Tensor:
    """``[B,C,T,H*p,W*p] -> [B,C*p*p,T,H,W]`` with channel order (c, column offset, row offset)."""
    if patch == 1:
        return x
    b, c, t, hh, ww = x.shape
    h, w = hh // patch, ww // patch
    x = x.reshape(b, c, t, h, patch, w, patch).permute(0, 1, 6, 4, 2, 3, 5)
    return x.reshape(b, c * patch * patch, t, h, w)


def pixel_unfold(x: torch.Tensor, patch: int = 2) -> torch.Tensor:
    """Inverse of :func:`pixel_fold`."""
    if patch == 1:
        return x
    b, cc, t, h, w = x.shape
    c = cc // (patch * patch)
    x = x.reshape(b, c, patch, patch, t, h, w).permute(0, 1, 4, 5, 3, 6, 2)
    return x.reshape(b, c, t, h * patch, w * patch)


def _channels_last(x: torch.Tensor) -> bool:
    """Whether a ``[B, C, T, H, W]`` tensor is laid out ``[B, T, H, W, C]`` in memory."""
    return x.ndim == 5 and x.permute(0, 2, 3, 4, 1).is_contiguous()


def _zeros_like_frames(x: torch.Tensor, frames: int) -> torch.Tensor:
    """``frames`` zero frames shaped like those of ``x``, in its memory layout (so that joining
    them with ``x`` along time keeps a channels-last volume channels-last)."""
    b, c, _, h, w = x.shape
    if _channels_last(x):
        return x.new_zeros(b, frames, h, w, c).permute(0, 4, 1, 2, 3)
    return x.new_zeros(b, c, frames, h, w)


class CausalConv3d(nn.Conv3d):
    """3-D convolution that never looks at later frames.

    Space is zero-padded by the convolution itself. In time the kernel sees ``kt - 1``
    earlier frames: those remembered in ``state`` when there are any, zeros otherwise.
    """

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0) -> None:
        def triple(v):
            return (v, v, v) if isinstance(v, int) else tuple(v)
        pad_t, pad_h, pad_w = triple(padding)
        super().__init__(in_channels, out_channels, triple(kernel_size), stride=triple(stride),
                         padding=(0, pad_h, pad_w))
        self.context = 2 * pad_t

    def forward(self, x: torch.Tensor, state: CausalState | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual`` is added to the result (inside the kernel when that runs)."""
        need = self.context
        if need == 0:
            return conv_volume(self, x, residual)
        previous = state.history.get(self) if state is not None else None
        if need == self.kernel_size[0] - 1 and eligible(self, x):
            # the kernel reads the remembered frames where they are (zeros before them)
            out = conv_volume_causal(self, x, previous, residual)
            if state is not None:
                have = 0 if previous is None else previous.shape[2]
                keep = min(_HISTORY, have + x.shape[2])
                recent = x if x.shape[2] >= keep else torch.cat([previous, x], dim=2)
                state.history[self] = recent[:, :, -keep:].clone()
            return out
        pieces = [x] if previous is None else [previous, x]
        have = 0 if previous is None else previous.shape[2]
        if have < need:
            pieces.insert(0, _zeros_like_frames(x, need - have))
        joined = torch.cat(pieces, dim=2)
        if state is not None:
            keep = min(_HISTORY, have + x.shape[2])
            state.history[self] = joined[:, :, -keep:].clone()
        return conv_volume(self, joined, residual)

    def plain(self, x: torch.Tensor) -> torch.Tensor:
        """The bare convolution, for callers that assemble the temporal context themselves."""
        return conv_volume(self, x)


class ChannelRMSNorm(nn.Module):
    """``x / ||x||_channels * sqrt(C) * gamma`` for channel-first maps, reduced in FP32."""

    def __init__(self, dim: int, *, images: bool = False) -> None:
        super().__init__()
        self.gain = float(dim) ** 0.5
        self.gamma = nn.Parameter(torch.ones(dim, *((1, 1) if images else (1, 1, 1))))

    def forward(self, x: torch.Tensor, silu: bool = False) -> torch.Tensor:
        """``silu=True`` applies the activation that follows every norm in the same pass."""
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.shape[1] <= 1024:
            from agentgarten_b200.ops import native

            if native.use(x):  # raises when the extension is missing on a GPU
                # channels-last activations are [pixels, C] rows: one fused kernel, one pass
                order = (0, *range(2, x.ndim), 1)
                rows = x.permute(order)
                if not rows.is_contiguous():
                    rows = rows.contiguous()
                native.count()
                out = native.ext().channel_norm(rows, self.gamma.detach().float().reshape(-1).contiguous(), silu)
                inverse = (0, x.ndim - 1, *range(1, x.ndim - 1))
                return out.permute(inverse)
        wide = x.float()
        norm = wide.norm(dim=1, keepdim=True).clamp_min(1e-12)
        out = wide * (self.gain / norm) * self.gamma.float()
        return (F.silu(out) if silu else out).to(x.dtype)


class ResidualBlock(nn.Module):
    """norm-SiLU-conv twice plus a (possibly projected) identity."""

    def __init__(self, in_dim: int, out_dim: int, dropout: float = 0.0) -> None:
        super().__init__()
        # Slots 1, 4 and 5 hold no parameters; they keep the checkpoint's numbering.
        self.residual = nn.Sequential(
            ChannelRMSNorm(in_dim), nn.SiLU(), CausalConv3d(in_dim, out_dim, 3, padding=1),
            ChannelRMSNorm(out_dim), nn.SiLU(), nn.Dropout(dropout),
            CausalConv3d(out_dim, out_dim, 3, padding=1))
        self.shortcut = CausalConv3d(in_dim, out_dim, 1) if in_dim != out_dim else nn.Identity()

    def forward(self, x: torch.Tensor, state: CausalState | None = None) -> torch.Tensor:
        r = self.residual
        h = r[2](r[0](x, silu=True), state)
        return r[6](r[5](r[3](h, silu=True)), state, residual=self.shortcut(x))


class FrameAttention(nn.Module):
    """Single-head self-attention over the pixels of each frame."""

    def __init__(self, dim: int) -> None:
        super().__init__()
        self.norm = ChannelRMSNorm(dim, images=True)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
        self.proj = nn.Conv2d(dim, dim, 1)
        nn.init.zeros_(self.proj.weight)

    def forward(self, x: torch.Tensor, state: CausalState | None = None) -> torch.Tensor:
        b, c, t, h, w = x.shape
        frames = x.transpose(1, 2).reshape(b * t, c, h, w)
        qkv = conv_frames(self.to_qkv, self.norm(frames)).reshape(b * t, 3, c, h * w).transpose(2, 3)
        mixed = F.scaled_dot_product_attention(qkv[:, 0:1], qkv[:, 1:2], qkv[:, 2:3])
        mixed = mixed.squeeze(1).transpose(1, 2).reshape(b * t, c, h, w)
        out = conv_frames(self.proj, mixed).reshape(b, t, c, h, w).transpose(1, 2)
        return x + out


class _FloatUpsample(nn.Upsample):
    """Nearest-exact 2x up-sampling of frames; parameter-free slot 0 of ``resample``."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.interpolate(x, scale_factor=(2.0, 2.0), mode="nearest-exact")


class Resample(nn.Module):
    """Spatial 2x re-sampling of every frame, optionally with a causal temporal 2x.

    ``mode`` is one of ``upsample2d``, ``upsample3d``, ``downsample2d``, ``downsample3d``.
    The temporal halves only act on chunks after the first: the first latent frame stands
    for a single pixel frame, every later one for four.
    """

    MODES = ("upsample2d", "upsample3d", "downsample2d", "downsample3d")

    def __init__(self, dim: int, mode: str) -> None:
        super().__init__()
        if mode not in self.MODES:
            raise ValueError(f"unknown resample mode {mode!r}")
        self.mode = mode
        if mode.startswith("up"):
            self.resample = nn.Sequential(_FloatUpsample(scale_factor=(2.0, 2.0), mode="nearest-exact"),
                                          nn.Conv2d(dim, dim, 3, padding=1))
            if mode == "upsample3d":
                self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
        else:
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=2))
            if mode == "downsample3d":
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=0)

    def _frames(self, x: torch.Tensor) -> torch.Tensor:
        b, c, t, h, w = x.shape
        y = conv_frames(self.resample[1], self.resample[0](x.transpose(1, 2).reshape(b * t, c, h, w)))
        return y.reshape(b, t, *y.shape[1:]).transpose(1, 2)

    def forward(self, x: torch.Tensor, state: CausalState | None = None) -> torch.Tensor:
        if self.mode == "upsample3d" and state is not None and not state.first:
            b, c, t, h, w = x.shape
            pair = self.time_conv(x, state)
            # Interleave the two predicted frames of every input frame along time.
            if _channels_last(pair):
                # [B, T, H, W, (2, C)] -> [B, (T, 2), H, W, C]: one copy, result channels-last
                rows = pair.permute(0, 2, 3, 4, 1).reshape(b, t, h, w, 2, c)
                x = rows.permute(0, 1, 4, 2, 3, 5).reshape(b, 2 * t, h, w, c).permute(0, 4, 1, 2, 3)
            else:
                x = pair.reshape(b, 2, c, t, h, w).permute(0, 2, 3, 1, 4, 5).reshape(b, c, 2 * t, h, w)
        x = self._frames(x)
        if self.mode == "downsample3d" and state is not None:
            last = x[:, :, -1:].clone()
            if not state.first:
                x = self.time_conv.plain(torch.cat([state.history[self], x], dim=2))
            state.history[self] = last
        return x


class AverageDown(nn.Module):
    """Parameter-free shortcut: fold a (time, row, column) block into channels, average groups."""

    def __init__(self, in_channels: int, out_channels: int, factor_t: int, factor_s: int) -> None:
        super().__init__()
        self.ft, self.fs = factor_t, factor_s
        folded = in_channels * factor_t * factor_s * factor_s
        if folded % out_channels:
            raise ValueError("folded channels must be a multiple of the output channels")
        self.out_channels, self.group = out_channels, folded // out_channels

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ft, fs = self.ft, self.fs
        lead = -x.shape[2] % ft
        if lead:
            x = torch.cat([_zeros_like_frames(x, lead), x], dim=2)
        b, c, t, h, w = x.shape
        if _channels_last(x):
            # [B, T, H, W, C] rows: gather each block behind its channel, average the groups;
            # the result is channels-last again.
            rows = x.permute(0, 2, 3, 4, 1).reshape(b, t // ft, ft, h // fs, fs, w // fs, fs, c)
            rows = rows.permute(0, 1, 3, 5, 7, 2, 4, 6).reshape(
                b, t // ft, h // fs, w // fs, self.out_channels, self.group)
            return rows.mean(dim=-1).permute(0, 4, 1, 2, 3)
        x = x.reshape(b, c, t // ft, ft, h // fs, fs, w // fs, fs).permute(0, 1, 3, 5, 7, 2, 4, 6)
        x = x.reshape(b, self.out_channels, self.group, t // ft, h // fs, w // fs)
        return x.mean(dim=2)


class DuplicateUp(nn.Module):
    """Parameter-free shortcut: repeat channels and unfold them into a (time, row, column) block."""

    def __init__(self, in_channels: int, out_channels: int, factor_t: int, factor_s: int) -> None:
        super().__init__()
        self.ft, self.fs = factor_t, factor_s
        unfolded = out_channels * factor_t * factor_s * factor_s
        if unfolded % in_channels:
            raise ValueError("unfolded channels must be a multiple of the input channels")
        self.out_channels, self.repeats = out_channels, unfolded // in_channels

    def forward(self, x: torch.Tensor, first: bool = False) -> torch.Tensor:
        ft, fs = self.ft, self.fs
        b, _, t, h, w = x.shape
        block = ft * fs * fs
        if _channels_last(x) and block % self.repeats == 0:
            # Channels-last volumes: output channel co at block offset k reads input channel
            # (co * block + k) // repeats = co * step + k // repeats, a strided slice; one copy
            # per block offset writes the result in place, channels-last.
            step = block // self.repeats
            rows = x.permute(0, 2, 3, 4, 1)
            out = rows.new_empty(b, t, ft, h, fs, w, fs, self.out_channels)
            for k in range(block):
                a, i, j = k // (fs * fs), (k // fs) % fs, k % fs
                out[:, :, a, :, i, :, j, :] = rows[..., k // self.repeats::step]
            out = out.view(b, t * ft, h * fs, w * fs, self.out_channels).permute(0, 4, 1, 2, 3)
            return out[:, :, ft - 1:] if first else out
        x = x.repeat_interleave(self.repeats, dim=1)
        x = x.reshape(b, self.out_channels, ft, fs, fs, t, h, w).permute(0, 1, 5, 2, 6, 3, 7, 4)
        x = x.reshape(b, self.out_channels, t * ft, h * fs, w * fs)
        return x[:, :, ft - 1:] if first else x


class DownStage(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, dropout: float, blocks: int, *, time: bool, space: bool) -> None:
        super().__init__()
        self.avg_shortcut = AverageDown(in_dim, out_dim, 2 if time else 1, 2 if space else 1)
        layers: list[nn.Module] = []
        for index in range(blocks):
            layers.append(ResidualBlock(in_dim if index == 0 else out_dim, out_dim, dropout))
        if space:
            layers.append(Resample(out_dim, "downsample3d" if time else "downsample2d"))
        self.downsamples = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor, state: CausalState | None = None) -> torch.Tensor:
        h = x
        for layer in self.downsamples:
            h = layer(h, state)
        return h + self.avg_shortcut(x)


class UpStage(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, dropout: float, blocks: int, *, time: bool, space: bool) -> None:
        super().__init__()
        self.avg_shortcut = DuplicateUp(in_dim, out_dim, 2 if time else 1, 2) if space else None
        layers: list[nn.Module] = []
        for index in range(blocks):
            layers.append(ResidualBlock(in_dim if index == 0 else out_dim, out_dim, dropout))
        if space:
            layers.append(Resample(out_dim, "upsample3d" if time else "upsample2d"))
        self.upsamples = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor, state: CausalState | None = None) -> torch.Tensor:
        h = x
        for layer in self.upsamples:
            h = layer(h, state)
        if self.avg_shortcut is None:
            return h
        return h + self.avg_shortcut(x, first=state is not None and state.first)


def _middle(dim: int, dropout: float) -> nn.Sequential:
    return nn.Sequential(ResidualBlock(dim, dim, dropout), FrameAttention(dim), ResidualBlock(dim, dim, dropout))


def _head(dim: int, out_channels: int) -> nn.Sequential:
    return nn.Sequential(ChannelRMSNorm(dim), nn.SiLU(), CausalConv3d(dim, out_channels, 3, padding=1))


class Encoder(nn.Module):
    def __init__(self, dim: int, out_channels: int, dim_mult: Sequence[int], blocks: int,
                 time_down: Sequence[bool], dropout: float, in_channels: int = 12) -> None:
        super().__init__()
        dims = [dim * m for m in (1, *dim_mult)]
        self.conv1 = CausalConv3d(in_channels, dims[0], 3, padding=1)
        stages = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            stages.append(DownStage(a, b, dropout, blocks, time=i < len(time_down) and bool(time_down[i]),
                                    space=i != len(dim_mult) - 1))
        self.downsamples = nn.Sequential(*stages)
        self.middle = _middle(dims[-1], dropout)
        self.head = _head(dims[-1], out_channels)

    def forward(self, x: torch.Tensor, state: CausalState | None = None) -> torch.Tensor:
        x = self.conv1(x, state)
        for stage in self.downsamples:
            x = stage(x, state)
        for layer in self.middle:
            x = layer(x, state)
        return self.head[2](self.head[0](x, silu=True), state)


class Decoder(nn.Module):
    def __init__(self, dim: int, in_channels: int, dim_mult: Sequence[int], blocks: int,
                 time_up: Sequence[bool], dropout: float, out_channels: int = 12) -> None:
        super().__init__()
        dims = [dim * m for m in (dim_mult[-1], *reversed(tuple(dim_mult)))]
        self.conv1 = CausalConv3d(in_channels, dims[0], 3, padding=1)
        self.middle = _middle(dims[0], dropout)
        stages = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            stages.append(UpStage(a, b, dropout, blocks + 1, time=i < len(time_up) and bool(time_up[i]),
                                  space=i != len(dim_mult) - 1))
        self.upsamples = nn.Sequential(*stages)
        self.head = _head(dims[-1], out_channels)

    def forward(self, x: torch.Tensor, state: CausalState | None = None) -> torch.Tensor:
        x = self.conv1(x, state)
        for layer in self.middle:
            x = layer(x, state)
        for stage in self.upsamples:
            x = stage(x, state)
        return self.head[2](self.head[0](x, silu=True), state)


class Wan22VAE(nn.Module):
    """Encoder, decoder and the two 1x1x1 latent projections of the Wan 2.2 VAE."""

    def __init__(self, dim: int = 160, dec_dim: int = 256, z_dim: int = 48,
                 dim_mult: Sequence[int] = (1, 2, 4, 4), num_res_blocks: int = 2,
                 temporal_downsample: Sequence[bool] = (False, True, True), dropout: float = 0.0,
                 patch: int = 2, image_channels: int = 3) -> None:
        super().__init__()
        self.z_dim, self.patch = z_dim, patch
        self.time_factor = 2 ** sum(bool(flag) for flag in temporal_downsample)
        folded = image_channels * patch * patch
        self.encoder = Encoder(dim, 2 * z_dim, dim_mult, num_res_blocks, temporal_downsample, dropout, folded)
        self.conv1 = CausalConv3d(2 * z_dim, 2 * z_dim, 1)
        self.conv2 = CausalConv3d(z_dim, z_dim, 1)
        self.decoder = Decoder(dec_dim, z_dim, dim_mult, num_res_blocks,
                               tuple(reversed(tuple(temporal_downsample))), dropout, folded)

    # ---- streaming primitives -------------------------------------------------------------
    def encode_chunk(self, pixels: torch.Tensor, state: CausalState) -> torch.Tensor:
        """Posterior mean of one chunk: a single frame first, then multiples of the time factor."""
        frames = pixels.shape[2]
        if state.first and frames != 1:
            raise ValueError("the first encoder chunk is exactly one frame")
        if not state.first and frames % self.time_factor:
            raise ValueError(f"later encoder chunks hold a multiple of {self.time_factor} frames")
        moments = self.conv1(self.encoder(pixel_fold(pixels, self.patch), state))
        state.advance()
        return moments[:, : self.z_dim]

    def decode_chunk(self, latent: torch.Tensor, state: CausalState) -> torch.Tensor:
        """Pixels of one chunk of (de-normalised) latent frames; the first chunk is one frame."""
        if state.first and latent.shape[2] != 1:
            raise ValueError("the first decoder chunk is exactly one latent frame")
        pixels = pixel_unfold(self.decoder(self.conv2(latent), state), self.patch)
        state.advance()
        return pixels

    # ---- whole clips -----------------------------------------------------------------------
    def encode(self, pixels: torch.Tensor, scale: tuple, *, temporal_window: int) -> torch.Tensor:
        """Normalised latent ``[B,z,1+(T-1)/4,H/16,W/16]`` of a clip of ``1`` or ``4n+1`` frames."""
        if isinstance(temporal_window, bool) or not isinstance(temporal_window, int) or temporal_window <= 0:
            raise ValueError(f"temporal_window must be a positive integer, got {temporal_window!r}")
        if temporal_window % self.time_factor:
            raise ValueError(f"temporal_window must be divisible by {self.time_factor}, got {temporal_window}")
        if pixels.ndim != 5:
            raise ValueError(f"Wan2.2 VAE input must be [B,C,T,H,W], got {tuple(pixels.shape)}")
        frames = int(pixels.shape[2])
        if frames != 1 and (frames - 1) % self.time_factor:
            raise ValueError(f"Wan2.2 VAE temporal length must be 1 or {self.time_factor}n+1, got {frames}")
        wanted = 1 + (frames - 1) // self.time_factor
        mean, inverse_std = (_per_channel(v, self.z_dim) for v in scale)
        state = CausalState()
        out = []
        for start in (0, *range(1, frames, temporal_window)):
            stop = 1 if start == 0 else start + temporal_window
            chunk = pixels[:, :, start:stop]
            short = (stop - start) - chunk.shape[2]
            if short:  # the last window is completed with blank frames and trimmed below
                chunk = torch.cat([chunk, chunk.new_zeros(*chunk.shape[:2], short, *chunk.shape[3:])], dim=2)
            out.append((self.encode_chunk(chunk, state) - mean) * inverse_std)
        return torch.cat(out, dim=2)[:, :, :wanted]

    def decode(self, latent: torch.Tensor, scale: tuple, *, frames_per_pass: int = 1) -> torch.Tensor:
        """Pixels ``[B,3,4T-3,16H,16W]`` of a normalised latent clip."""
        mean, inverse_std = (_per_channel(v, self.z_dim) for v in scale)
        latent = latent / inverse_std + mean
        state = CausalState()
        out = [self.decode_chunk(latent[:, :, :1], state)]
        step = max(1, int(frames_per_pass))
        for start in range(1, latent.shape[2], step):
            out.append(self.decode_chunk(latent[:, :, start:start + step], state))
        return torch.cat(out, dim=2) if len(out) > 1 else out[0]


@torch.no_grad()
def to_channels_last(module: nn.Module) -> nn.Module:
    """Convolution weights in the layout of the tensor-core kernels: 5-D -> NDHWC, 4-D -> NHWC."""
    for parameter in module.parameters():
        if parameter.ndim == 5:
            parameter.data = parameter.data.contiguous(memory_format=torch.channels_last_3d)
        elif parameter.ndim == 4 and parameter.shape[-1] * parameter.shape[-2] > 1:
            parameter.data = parameter.data.contiguous(memory_format=torch.channels_last)
    return module


def _per_channel(value, channels: int):
    if isinstance(value, torch.Tensor):
        return value.view(1, channels, 1, 1, 1)
    return value


def build_vae(pretrained_path: str | Path | None = None, *, device: str | torch.device = "cpu",
              **overrides) -> Wan22VAE:
    """Construct on the meta device, then adopt the checkpoint's tensors (or leave storage empty).

    Loading is local to the calling rank: the codec is created lazily by whichever rank
    owns the raw batch, so a collective here would wait on ranks that never enter it.
    """
    with torch.device("meta"):
        model = Wan22VAE(**overrides)
    if pretrained_path is None:
        return model.to_empty(device=device)
    prefetch(pretrained_path)
    log.info(f"loading {pretrained_path}")
    weights = torch.load(pretrained_path, map_location=device, weights_only=True, mmap=True)
    if isinstance(weights, dict) and "state_dict" in weights:
        weights = weights["state_dict"]
    model.load_state_dict(weights, assign=True)
    return model


def random_vae(*, seed: int = 0, device: str | torch.device = "cpu", **overrides) -> Wan22VAE:
    """A VAE with reproducible random weights, for tests and synthetic benchmarks."""
    model = Wan22VAE(**overrides).to(device)
    generator = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.ndim > 1 and not name.endswith("gamma"):
                fan_in = p[0].numel()
                p.copy_(torch.randn(p.shape, generator=generator) * math.sqrt(1.0 / fan_in))
            elif name.endswith("bias"):
                p.copy_(torch.randn(p.shape, generator=generator) * 0.02)
    return model


_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
# Pixel frames per encoder window by the shorter image side: bounds activation memory while
# keeping each pass large enough to fill the GPU.
_ENCODE_WINDOW = ((256, 68), (640, 24), (None, 12))
# Latent frames the decoder advances per pass after the first, by latent pixels per frame.
_DECODE_BUDGET = 4 * 45 * 80


class Wan22VAECodec:
    """Lazy, frozen Wan 2.2 codec: ``encode`` pixels in [-1,1] to normalised latents and back.

    The weights are materialised on first use, on the device of the first tensor seen (or
    ``device``). ``decoder`` optionally replaces the native decoder by a lighter one with
    the same latent space; encoding always uses the native encoder.
    """

    def __init__(self, pretrained_path: str | Path | None, *, dtype: torch.dtype | str = "bfloat16",
                 device: torch.device | str | None = None, temporal_compression_factor: int = 4,
                 decoder=None, architecture: dict | None = None) -> None:
        self.pretrained_path = None if pretrained_path is None else str(pretrained_path)
        self.decoder = decoder
        self.dtype = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        self.preferred_device = None if device is None else torch.device(device)
        self.temporal_compression_factor = int(temporal_compression_factor)
        self.architecture = dict(architecture or {})
        self._vae: Wan22VAE | None = None
        self._scale: tuple[torch.Tensor, torch.Tensor] | None = None

    # ---- lazily shared pieces ------------------------------------------------------------
    def _get_vae(self, device: torch.device | str | None = None) -> Wan22VAE:
        if self._vae is None:
            target = self.preferred_device if device is None else torch.device(device)
            target = target or torch.device("cpu")
            if self.pretrained_path is None:
                vae = random_vae(device=target, **self.architecture)
            else:
                vae = build_vae(self.pretrained_path, device=target, **self.architecture)
            vae = vae.eval().requires_grad_(False).to(dtype=self.dtype)
            if target.type == "cuda":
                vae = to_channels_last(vae)
            self._vae = vae
        return self._vae

    def _normalization(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
        if self._scale is None or self._scale[0].device != device:
            channels = self.latent_channels
            mean = torch.tensor(LATENT_MEAN[:channels], dtype=self.dtype, device=device)
            std = torch.tensor(LATENT_STD[:channels], dtype=self.dtype, device=device)
            self._scale = mean, 1.0 / std
        return self._scale

    def stream_components(self, device: torch.device | str) -> tuple[nn.Module, tuple[torch.Tensor, torch.Tensor]]:
        """The shared frozen VAE and its normalisation, for an online codec.

        Streaming callers own their recurrence (:class:`CausalState`) and must not interleave
        with full-clip calls on the same CUDA stream ordering assumptions; the weights are
        read-only, so any number of streams may share them.
        """
        device = torch.device(device)
        return self._get_vae(device), self._normalization(device)

    def stream(self, device: torch.device | str) -> "Wan22Stream":
        return Wan22Stream(*self.stream_components(device), dtype=self.dtype)

    @staticmethod
    def _encode_window(spatial_shape: Sequence[int]) -> int:
        shorter = min(int(v) for v in spatial_shape)
        for limit, frames in _ENCODE_WINDOW:
            if limit is None or shorter <= limit:
                return frames
        raise AssertionError("unreachable")

    @staticmethod
    def _decode_frames_per_pass(latent_shape: Sequence[int]) -> int:
        per_frame = int(latent_shape[-1]) * int(latent_shape[-2]) * int(latent_shape[0])
        return max(1, _DECODE_BUDGET // max(1, per_frame))

    # ---- public surface --------------------------------------------------------------------
    @torch.no_grad()
    def encode(self, video: torch.Tensor) -> torch.Tensor:
        if not video.is_floating_point():
            raise TypeError("Wan 2.2 VAE input must be floating point")
        vae = self._get_vae(video.device)
        with torch.autocast(device_type=video.device.type, enabled=False):
            latent = vae.encode(video.to(self.dtype), self._normalization(video.device),
                                temporal_window=self._encode_window(video.shape[-2:]))
        return latent.to(video.dtype)

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        if not latent.is_floating_point():
            raise TypeError("Wan 2.2 VAE latent must be floating point")
        if self.decoder is not None:
            return self.decoder.decode(latent)
        vae = self._get_vae(latent.device)
        with torch.autocast(device_type=latent.device.type, enabled=False):
            video = vae.decode(latent.to(self.dtype), self._normalization(latent.device),
                               frames_per_pass=self._decode_frames_per_pass(latent.shape))
        return video.to(latent.dtype)

    @property
    def spatial_compression_factor(self) -> int:
        return 16

    @property
    def latent_channels(self) -> int:
        return int(self.architecture.get("z_dim", 48))

    def latent_frames(self, pixel_frames: int) -> int:
        return (int(pixel_frames) - 1) // self.temporal_compression_factor + 1

    def pixel_frames(self, latent_frames: int) -> int:
        return (int(latent_frames) - 1) * self.temporal_compression_factor + 1


class Wan22Stream:
    """Online encode/decode on shared weights: each direction keeps its own recurrence.

    ``encode`` takes the first pixel frame alone and then any multiple of four frames;
    ``decode`` takes one latent frame first and then any number per call, returning one
    pixel frame for the first latent frame and four for each later one.
    """

    def __init__(self, vae: Wan22VAE, scale: tuple[torch.Tensor, torch.Tensor], *, dtype: torch.dtype) -> None:
        self.vae, self.scale, self.dtype = vae, scale, dtype
        self._encoder, self._decoder = CausalState(), CausalState()

    def reset(self) -> None:
        self._encoder.reset()
        self._decoder.reset()

    @torch.no_grad()
    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        mean, inverse_std = (_per_channel(v, self.vae.z_dim) for v in self.scale)
        pieces = []
        source = pixels.to(self.dtype)
        if self._encoder.first:
            pieces.append(self.vae.encode_chunk(source[:, :, :1], self._encoder))
            source = source[:, :, 1:]
        if source.shape[2]:
            pieces.append(self.vae.encode_chunk(source, self._encoder))
        return ((torch.cat(pieces, dim=2) - mean) * inverse_std).to(pixels.dtype)

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        mean, inverse_std = (_per_channel(v, self.vae.z_dim) for v in self.scale)
        source = latent.to(self.dtype) / inverse_std + mean
        pieces = []
        if self._decoder.first:
            pieces.append(self.vae.decode_chunk(source[:, :, :1], self._decoder))
            source = source[:, :, 1:]
        if source.shape[2]:
            pieces.append(self.vae.decode_chunk(source, self._decoder))
        return torch.cat(pieces, dim=2).to(latent.dtype)
