"""Depth/normal preprocessing: colourisation, normal preparation, pooling, robustness
augmentations (texture suppression, warp that fades out from the first frame, modality
dropout/selection) and the quadrant stretch to a VAE-friendly size.

Everything here is plain tensor arithmetic on ``[B, C, T, H, W]`` videos; no graphics API.
Random decisions are drawn on the CPU generator in a fixed order (texture: applied,
factor; warp: applied, log-scales, shifts, shears, perspective; dropout: choice, drop;
stretch: top, left), so a seeded run is reproducible on any device.

Parity: reference ``wm/networks/cosmos3/geometry.py:31-644``.
"""

from __future__ import annotations

import hashlib
import math
from collections.abc import Mapping
from dataclasses import dataclass
from enum import StrEnum
from typing import Any

import torch
import torch.nn.functional as F

__all__ = [
    "GeometryAugmentationConfig",
    "GeometryKind",
    "ModalitySelection",
    "augment_geometry",
    "colorize_depth",
    "depth_scale",
    "downsample_geometry",
    "prepare_normal",
    "stretch_geometry",
]


class GeometryKind(StrEnum):
    DEPTH = "depth"
    NORMAL = "normal"


class ModalitySelection(StrEnum):
    BOTH = "both"
    RANDOM_SINGLE = "random_single"
    DEPTH = "depth"
    NORMAL = "normal"


_SLOTS = (GeometryKind.DEPTH, GeometryKind.NORMAL)


def _finite(value: float) -> bool:
    return math.isfinite(float(value))


@dataclass(frozen=True, slots=True)
class GeometryAugmentationConfig:
    modality_dropout_probability: float = 0.0
    modality_selection: ModalitySelection | str = "both"
    spatial_probability: float = 0.0
    spatial_max_scale: float = 1.0
    spatial_max_shift_fraction: float = 0.0
    spatial_max_shear: float = 0.0
    spatial_max_perspective: float = 0.0
    spatial_anneal_power: float = 1.0
    texture_suppression_probability: float = 0.0
    texture_downsample_min: float = 1.0
    texture_downsample_max: float = 1.0
    texture_gaussian_sigma_scale: float = 0.5
    texture_skip_tsdf: bool = True
    geometry_spatial_downsample: int = 4
    geometry_stretch_divisor: int = 32

    def __post_init__(self) -> None:
        object.__setattr__(self, "modality_selection", ModalitySelection(self.modality_selection))
        for name in ("modality_dropout_probability", "spatial_probability",
                     "texture_suppression_probability"):
            v = getattr(self, name)
            if not _finite(v) or not 0.0 <= v <= 1.0:
                raise ValueError(f"{name} must be finite and in [0, 1]")
        if not _finite(self.spatial_max_scale) or self.spatial_max_scale < 1.0:
            raise ValueError("spatial_max_scale must be finite and at least one")
        for name, top in (("spatial_max_shift_fraction", 0.5), ("spatial_max_shear", 0.5),
                          ("spatial_max_perspective", 0.25)):
            v = getattr(self, name)
            if not _finite(v) or not 0.0 <= v <= top:
                raise ValueError(f"{name} must be finite and in [0, {top}]")
        if not _finite(self.spatial_anneal_power) or self.spatial_anneal_power <= 0:
            raise ValueError("spatial_anneal_power must be finite and positive")
        lo, hi = self.texture_downsample_min, self.texture_downsample_max
        if not (_finite(lo) and _finite(hi)) or lo < 1.0 or hi < lo:
            raise ValueError("texture downsample range must be finite, ordered, and at least one")
        if not _finite(self.texture_gaussian_sigma_scale) or self.texture_gaussian_sigma_scale < 0:
            raise ValueError("texture_gaussian_sigma_scale must be finite and non-negative")
        if int(self.geometry_spatial_downsample) <= 0:
            raise ValueError("geometry_spatial_downsample must be positive")
        if int(self.geometry_stretch_divisor) <= 0:
            raise ValueError("geometry_stretch_divisor must be positive")


# ------------------------------------------------------------------ colourisation
def _fused_kernels(tensor: torch.Tensor):
    """The CUDA extension when ``tensor`` lives on a GPU and no gradient is wanted (one-pass
    kernels of ``csrc/geometry.cu``), else ``None``."""
    if not tensor.is_cuda or (torch.is_grad_enabled() and tensor.requires_grad):
        return None
    from agentgarten_b200.ops import native

    if not native.use(tensor, dtypes=(tensor.dtype,)):  # raises when the extension is missing
        return None
    native.count()
    return native.ext()


def colorize_depth(depth: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Metric depth ``[B,1,T,H,W]`` → RGB in [0,1] along a 7-segment walk on the colour
    cube.  ``t = 1 - (1 + d·s/10)^-2`` compresses far depth; invalid pixels are black."""
    fused = _fused_kernels(depth)
    if fused is not None and depth.dtype == torch.float32 and depth.ndim == 5 and depth.shape[1] == 1:
        weights = scale.to(device=depth.device, dtype=torch.float32).reshape(-1).contiguous()
        if weights.shape[0] in (1, depth.shape[0]):
            return fused.colorize_depth(depth.contiguous(), weights)
    valid = torch.isfinite(depth) & (depth > 0)
    safe = torch.where(valid, depth.clamp_min(0.0), 0.0)
    scale = scale.to(device=depth.device, dtype=torch.float32).reshape(-1)
    if scale.shape[0] == 1 and depth.shape[0] != 1:
        scale = scale.expand(depth.shape[0])
    t = 1.0 - (1.0 + safe * scale.view(-1, 1, 1, 1, 1) / 10.0).pow(-2.0)
    t = torch.where(valid, t.clamp(0.0, 1.0), 0.0)
    s = t[:, 0] * 7.0

    def ramp(offset: float) -> torch.Tensor:
        return (s - offset).clamp(0.0, 1.0)

    red = ramp(0.0) - ramp(2.0) + ramp(5.0)
    green = ramp(1.0) - ramp(4.0) + ramp(6.0)
    blue = ramp(3.0)
    rgb = torch.stack((red, green, blue), dim=1)
    return rgb.masked_fill(~valid.expand(-1, 3, -1, -1, -1), 0.0)


def prepare_normal(normal: torch.Tensor) -> torch.Tensor:
    """uint8 normals are decoded to [-1,1] and re-normalised (degenerate → 0); float normals
    are trusted as they are (a second normalisation would perturb every VAE input)."""
    if normal.dtype == torch.uint8:
        fused = _fused_kernels(normal)
        if fused is not None and normal.ndim == 5 and normal.shape[1] == 3:
            return fused.decode_normal(normal.contiguous())
        n = normal.float() / 127.5 - 1.0
        finite = torch.isfinite(n).all(dim=1, keepdim=True)
        n = n.nan_to_num(nan=0.0, posinf=0.0, neginf=0.0)
        tiny = torch.finfo(torch.float32).eps
        length = torch.linalg.vector_norm(n, dim=1, keepdim=True)
        ok = finite & (length > tiny)
        n = n / length.clamp_min(tiny)
        return n.masked_fill(~ok.expand_as(n), 0.0).contiguous()
    if not normal.is_floating_point():
        raise TypeError(f"raw normal must be uint8 or floating point, got {normal.dtype}")
    return normal.to(dtype=torch.float32, copy=True).contiguous()


def _frames_as_images(video: torch.Tensor) -> torch.Tensor:
    b, c, t, h, w = video.shape
    return video.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)


def _images_as_frames(images: torch.Tensor, batch: int) -> torch.Tensor:
    bt, c, h, w = images.shape
    return images.reshape(batch, bt // batch, c, h, w).permute(0, 2, 1, 3, 4)


def downsample_geometry(videos: Mapping[str, torch.Tensor], *, factor: int) -> dict[str, torch.Tensor]:
    out = {}
    for name, video in videos.items():
        fused = _fused_kernels(video) if video.dtype == torch.float32 else None
        if fused is not None:
            out[name] = fused.pool_frames(video.contiguous(), factor)  # cleans and pools in one pass
            continue
        clean = torch.nan_to_num(video, nan=0.0, posinf=0.0, neginf=0.0)
        low = F.avg_pool2d(_frames_as_images(clean), kernel_size=factor, stride=factor)
        out[name] = _images_as_frames(low, video.shape[0]).contiguous()
    return out


# ------------------------------------------------------------------ augmentations
def _flag(batch: Mapping[str, Any], key: str, size: int) -> torch.Tensor:
    value = batch.get(key)
    if value is None:
        return torch.zeros(size, dtype=torch.bool)
    flag = torch.as_tensor(value, device="cpu", dtype=torch.bool).reshape(-1)
    if flag.numel() == 1 and size != 1:
        flag = flag.expand(size)
    if flag.numel() != size:
        raise ValueError(f"{key} must contain one flag per sample, got {flag.numel()} "
                         f"for batch size {size}")
    return flag


def _gaussian(images: torch.Tensor, sigma: float) -> torch.Tensor:
    if sigma <= 0:
        return images
    radius = max(1, math.ceil(3.0 * sigma))
    x = torch.arange(-radius, radius + 1, device=images.device, dtype=images.dtype)
    kernel = torch.exp(-0.5 * x.square() / (sigma * sigma))
    kernel = kernel / kernel.sum()
    fused = _fused_kernels(images) if images.dtype == torch.float32 else None
    if fused is not None:
        return fused.blur_frames(images.contiguous(), kernel.contiguous())  # no padded copies
    c = images.shape[1]
    rows = kernel.view(1, 1, 1, -1).repeat(c, 1, 1, 1)
    cols = kernel.view(1, 1, -1, 1).repeat(c, 1, 1, 1)
    out = F.conv2d(F.pad(images, (radius, radius, 0, 0), mode="replicate"), rows, groups=c)
    return F.conv2d(F.pad(out, (0, 0, radius, radius), mode="replicate"), cols, groups=c)


def _suppress_texture(videos, *, data_batch, config) -> dict[str, torch.Tensor]:
    """Per sample: Gaussian prefilter → area downsample → bilinear upsample."""
    first = next(iter(videos.values()))
    b, _, _, h, w = first.shape
    p = config.texture_suppression_probability
    if p <= 0:
        return dict(videos)
    applied = torch.rand(b, device="cpu") < p
    if config.texture_skip_tsdf:
        applied &= ~_flag(data_batch, "geometry_condition_is_augmented", b)
    if not bool(applied.any()):
        return dict(videos)
    u = torch.rand(b, device="cpu")
    factors = config.texture_downsample_min + (
        config.texture_downsample_max - config.texture_downsample_min) * u
    names = tuple(videos)
    widths = [int(videos[n].shape[1]) for n in names]
    out = {n: v.clone() for n, v in videos.items()}
    for i in torch.nonzero(applied).flatten().tolist():
        f = float(factors[i])
        images = torch.cat([videos[n][i].permute(1, 0, 2, 3) for n in names], dim=1)
        images = _gaussian(images, f * config.texture_gaussian_sigma_scale)
        low_size = (max(1, round(h / f)), max(1, round(w / f)))
        fused = _fused_kernels(images) if images.dtype == torch.float32 else None
        if fused is not None:
            low = fused.resize_frames(images.contiguous(), *low_size, True)
            smooth = fused.resize_frames(low, h, w, False)
        else:
            low = F.interpolate(images, size=low_size, mode="area")
            smooth = F.interpolate(low, size=(h, w), mode="bilinear", align_corners=False)
        for n, part in zip(names, smooth.split(widths, dim=1), strict=True):
            out[n][i].copy_(part.permute(1, 0, 2, 3))
    return out


def _warp_from_first_frame(videos, *, config) -> dict[str, torch.Tensor]:
    """Random scale/shift/shear/perspective whose strength fades from frame 0 to the last
    frame (``(1 - progress)^power``), sampled with bilinear ``grid_sample``."""
    first = next(iter(videos.values()))
    b, _, t, h, w = first.shape
    applied = torch.zeros(b, dtype=torch.bool)
    if config.spatial_probability > 0:
        applied = torch.rand(b, device="cpu") < config.spatial_probability
    if not bool(applied.any()):
        return dict(videos)

    def draw(bound: float) -> torch.Tensor:
        value = (torch.rand((b, 2), device="cpu") * 2.0 - 1.0) * bound
        return torch.where(applied[:, None], value, torch.zeros_like(value))

    log_scale = draw(math.log(config.spatial_max_scale))
    shift = draw(config.spatial_max_shift_fraction)
    shear = draw(config.spatial_max_shear)
    persp = draw(config.spatial_max_perspective)
    device, dtype = first.device, torch.float32
    ys = (torch.arange(h, device=device, dtype=dtype) + 0.5) * (2.0 / h) - 1.0
    xs = (torch.arange(w, device=device, dtype=dtype) + 0.5) * (2.0 / w) - 1.0
    gy, gx = torch.meshgrid(ys, xs, indexing="ij")
    gx, gy = gx[None, None], gy[None, None]
    if t == 1:
        strength = torch.ones((1, 1, 1, 1), device=device, dtype=dtype)
    else:
        progress = torch.linspace(0.0, 1.0, t, device=device, dtype=dtype)
        strength = (1.0 - progress).pow(config.spatial_anneal_power)[None, :, None, None]

    def col(value: torch.Tensor, index: int) -> torch.Tensor:
        return value[:, index].to(device=device, dtype=dtype)[:, None, None, None]

    sx, sy = (strength * col(log_scale, 0)).exp(), (strength * col(log_scale, 1)).exp()
    tx, ty = strength * col(shift, 0) * 2.0, strength * col(shift, 1) * 2.0
    hx, hy = strength * col(shear, 0), strength * col(shear, 1)
    px, py = strength * col(persp, 0), strength * col(persp, 1)
    stacked_input = torch.cat([videos[n] for n in videos], dim=1)
    fused = _fused_kernels(stacked_input) if stacked_input.dtype == torch.float32 else None
    if fused is not None:
        # one kernel: the map of every frame from its eight numbers, bilinear sampling with border
        # clamping, the unchanged last frame and the samples that are not warped
        terms = [term.expand(b, t, 1, 1).reshape(b, t) for term in (sx, sy, tx, ty, hx, hy, px, py)]
        keep = (~applied).to(device)[:, None].expand(b, t).clone()
        if t > 1:
            keep[:, -1] = True
        warped = fused.warp_frames(stacked_input.contiguous(), torch.stack(terms, dim=-1).contiguous(),
                                   keep.to(torch.uint8).contiguous())
        names = tuple(videos)
        return dict(zip(names, warped.split([int(videos[n].shape[1]) for n in names], dim=1), strict=True))
    denom = (1.0 + px * gx + py * gy).clamp_min(0.5)
    src_x = (sx * gx + hx * gy + tx) / denom
    src_y = (hy * gx + sy * gy + ty) / denom
    grid = torch.stack((src_x, src_y), dim=-1).reshape(b * t, h, w, 2)
    names = tuple(videos)
    widths = [int(videos[n].shape[1]) for n in names]
    stacked = torch.cat([videos[n] for n in names], dim=1)
    warped = F.grid_sample(_frames_as_images(stacked), grid, mode="bilinear",
                           padding_mode="border", align_corners=False)
    warped = _images_as_frames(warped, b).clone()
    if t > 1:
        warped[:, :, -1] = stacked[:, :, -1]  # exact identity at the last frame
    if not bool(applied.all()):
        warped = torch.where(applied.to(device)[:, None, None, None, None], warped, stacked)
    return dict(zip(names, warped.split(widths, dim=1), strict=True))


def _drop_modality(videos, *, config, apply_dropout: bool = True,
                   validation_choices: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
    """Blank whole modalities: both with ``modality_dropout_probability``; under a
    single-modality selection the *other* modality always."""
    first = next(iter(videos.values()))
    b = int(first.shape[0])
    p, selection = config.modality_dropout_probability, config.modality_selection
    names = tuple(n for n in _SLOTS if n in videos)
    if not names or (selection is ModalitySelection.BOTH and p <= 0):
        return dict(videos)
    blank = torch.zeros((b, 2), dtype=torch.bool)
    if selection is not ModalitySelection.BOTH:
        if set(names) != set(_SLOTS):
            raise ValueError("single-modality selection requires both raw geometry slots")
        if selection is ModalitySelection.RANDOM_SINGLE:
            choice = torch.randint(2, (b,), device="cpu") if validation_choices is None \
                else validation_choices
        else:
            other = GeometryKind.NORMAL if selection is ModalitySelection.DEPTH else GeometryKind.DEPTH
            choice = torch.full((b,), names.index(other))
        blank[torch.arange(b), choice] = True
    if apply_dropout and p > 0:
        everything = torch.rand(b, device="cpu") < p
        for n in names:
            blank[:, _SLOTS.index(n)] |= everything
    out = dict(videos)
    for n in names:
        chosen = blank[:, 0 if n is GeometryKind.DEPTH else 1]
        if not bool(chosen.any()):
            continue
        video = videos[n]
        if int(video.shape[1]) != 3:
            raise ValueError(f"prepared {n} must have three color channels before dropout")
        # depth colours live in [0,1], normals in [-1,1]: both become -1 at the VAE input
        fill = video.new_tensor(0.0 if n is GeometryKind.DEPTH else -1.0)
        out[n] = torch.where(chosen.to(first.device)[:, None, None, None, None], fill, video).contiguous()
    return out


def _validation_choices(data_batch: Mapping[str, Any], size: int) -> torch.Tensor:
    """Deterministic per-sample modality for validation: one bit of a SHA-256 digest."""

    def rows(value: Any) -> list[Any]:
        if torch.is_tensor(value):
            value = value.detach().cpu().reshape(-1).tolist()
        elif isinstance(value, (str, int)):
            value = [value] * size
        else:
            value = list(value)
        if len(value) != size:
            raise ValueError("validation modality metadata must match batch size")
        return value

    keys = rows(data_batch.get("__key__", data_batch.get("validation_manifest_slot", range(size))))
    seeds = rows(data_batch.get("validation_sample_seed", 0))
    bits = [hashlib.sha256(f"cosmos3-validation-modality-v1:{int(s)}:{k}".encode()).digest()[0] & 1
            for k, s in zip(keys, seeds, strict=True)]
    return torch.tensor(bits, dtype=torch.long)


def augment_geometry(videos, *, data_batch, training: bool, config) -> dict[str, torch.Tensor]:
    if not videos:
        return dict(videos)
    if not training:
        if config.modality_selection is ModalitySelection.BOTH:
            return dict(videos)
        choices = None
        if config.modality_selection is ModalitySelection.RANDOM_SINGLE:
            choices = _validation_choices(data_batch, int(next(iter(videos.values())).shape[0]))
        return _drop_modality(videos, config=config, apply_dropout=False, validation_choices=choices)
    smooth = _suppress_texture(videos, data_batch=data_batch, config=config)
    warped = _warp_from_first_frame(smooth, config=config)
    return _drop_modality(warped, config=config)


def stretch_geometry(videos, *, training: bool, divisor: int) -> dict[str, torch.Tensor]:
    """Grow each video to the next multiple of ``divisor`` by bilinearly stretching its four
    quadrants around the centre; the extra rows/columns are split randomly between the two
    sides in training and evenly at evaluation."""
    first = next(iter(videos.values()))
    b, _, _, h, w = first.shape
    th, tw = -(-h // divisor) * divisor, -(-w // divisor) * divisor
    extra_h, extra_w = th - h, tw - w
    if training:
        tops = torch.randint(0, extra_h + 1, (b,), device="cpu")
        lefts = torch.randint(0, extra_w + 1, (b,), device="cpu")
    else:
        tops = torch.full((b,), extra_h // 2, dtype=torch.long)
        lefts = torch.full((b,), extra_w // 2, dtype=torch.long)
    names = tuple(videos)
    widths = [int(videos[n].shape[1]) for n in names]
    fused = _fused_kernels(first) if first.dtype == torch.float32 and min(h, w) >= 2 else None
    if fused is not None and all(videos[n].dtype == torch.float32 for n in names):
        # one kernel for all samples and modalities: both resizes of every quadrant, no pieces
        stacked = torch.cat([videos[n] for n in names], dim=1).contiguous()
        grown = fused.stretch_frames(stacked, tops.to(first.device, torch.int32),
                                     lefts.to(first.device, torch.int32), th, tw)
        return dict(zip(names, grown.split(widths, dim=1), strict=True))
    rows: dict[str, list[torch.Tensor]] = {n: [] for n in names}
    up, left_w = h // 2, w // 2
    down, right_w = h - up, w - left_w

    def resize(x, size):
        return F.interpolate(x, size=size, mode="bilinear", align_corners=False)

    for i in range(b):
        top, left = int(tops[i]), int(lefts[i])
        images = torch.cat([videos[n][i].permute(1, 0, 2, 3) for n in names], dim=1)
        a, c = images.split((up, down), dim=-2)
        images = torch.cat((resize(a, (up + top, w)), resize(c, (down + extra_h - top, w))), dim=-2)
        a, c = images.split((left_w, right_w), dim=-1)
        images = torch.cat((resize(a, (th, left_w + left)),
                            resize(c, (th, right_w + extra_w - left))), dim=-1)
        for n, part in zip(names, images.split(widths, dim=1), strict=True):
            rows[n].append(part.permute(1, 0, 2, 3).unsqueeze(0))
    return {n: torch.cat(parts, dim=0) for n, parts in rows.items()}


def depth_scale(data_batch: Mapping[str, Any], *, training: bool, batch_size: int | None = None,
                scale_key: str = "depth_scale", eligible_key: str = "depth_scale_jitter_eligible",
                bounds_key: str = "depth_scale_jitter_bounds") -> torch.Tensor:
    """Per-sample depth scale, multiplied in training by a uniform factor from
    ``bounds`` for samples marked eligible."""
    scale = torch.as_tensor(data_batch[scale_key])
    if scale.ndim == 0 or scale.numel() == 0:
        raise ValueError("depth scale must contain one value per batch")
    if scale.is_complex():
        raise TypeError("depth scale must be real-valued")
    if not scale.is_floating_point():
        scale = scale.float()
    scale = scale.reshape(-1)
    if batch_size is not None and scale.numel() not in (1, int(batch_size)):
        raise ValueError(f"depth scale must have batch size 1 or {batch_size}, got {scale.numel()}")
    if not torch.isfinite(scale).all() or (scale <= 0).any():
        raise ValueError("depth scale must be finite and positive")
    eligible, bounds = data_batch.get(eligible_key), data_batch.get(bounds_key)
    if not (training and eligible is not None and bounds is not None):
        return scale
    n = int(scale.shape[0])
    eligible = torch.as_tensor(eligible, device=scale.device, dtype=torch.bool)
    bounds = torch.as_tensor(bounds, device=scale.device, dtype=torch.float32)
    if eligible.numel() not in (1, n):
        raise ValueError(f"depth scale jitter eligibility must have batch size 1 or {n}, "
                         f"got {eligible.numel()}")
    if bounds.ndim != 2 or bounds.shape[1] != 2 or bounds.shape[0] not in (1, n):
        raise ValueError(f"depth scale jitter bounds must have shape [1, 2] or [{n}, 2], "
                         f"got {tuple(bounds.shape)}")
    bounds = bounds.expand(n, -1) if bounds.shape[0] == 1 else bounds
    eligible = eligible.expand(n) if eligible.numel() == 1 else eligible.reshape(-1)
    if not torch.isfinite(bounds).all() or (bounds[:, 1] < bounds[:, 0]).any():
        raise ValueError("depth scale jitter bounds must be finite and ordered")
    u = torch.rand((n,), device="cpu").to(scale.device)
    factor = torch.where(eligible, bounds[:, 0] + (bounds[:, 1] - bounds[:, 0]) * u,
                         torch.ones_like(u))
    return scale * factor.to(scale.dtype)
