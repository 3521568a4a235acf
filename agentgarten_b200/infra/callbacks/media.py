"""Writing sampled clips as images / videos.

A sample is a mapping of named videos (``depth``, ``normal``, ``ground_truth``, ``sample``)
in ``[B, C, T, H, W]`` (or ``[B, T, C, H, W]``) layout with values in [-1, 1] (or [0, 1], or
uint8).  Tensors are converted to uint8 on the host in frame chunks; an optional grid tiles
three (1x3) or four (2x2) of them, resizing the condition panels to the reference panel.
One-frame results are stored as images, longer ones as videos; files are written atomically
as ``Iter%09d_Rank%04d_<name>_<batch>[_<index>].<ext>``, optionally from a background
thread (one write in flight; a failure disables the writer).

Parity: reference ``wm/infra/callbacks/media.py:23-486``.
"""

from __future__ import annotations

from collections.abc import Iterator, Mapping, Sequence
from threading import Thread
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor

from agentgarten_b200.utils import io, log

__all__ = ["ImageVideoArtifactWriter", "media_artifact_filename", "video_batch_to_cpu_uint8"]


def _safe(value: Any) -> str:
    text = "".join(c if c.isalnum() or c in "-_." else "_" for c in str(value))
    return text.strip("._") or "sample"


def media_artifact_filename(*, artifact_name: str, iteration: int, rank: int, sample_batch_index: int,
                            extension: str, batch_index: int | None = None) -> str:
    numbers = (int(sample_batch_index),) + (() if batch_index is None else (int(batch_index),))
    tail = "_".join(f"{n:02d}" for n in numbers)
    # as the reference writes them: the indices follow the name directly, with an "@" in between
    # only when an index needs three digits (``wm/infra/callbacks/media.py:112-129``)
    joiner = "@" if any(n >= 100 for n in numbers) else ""
    return f"Iter{int(iteration):09d}_Rank{int(rank):04d}_{_safe(artifact_name)}{joiner}{tail}.{extension}"


def _canonical(video: Tensor, layout: str) -> Tensor:
    """-> ``[B, 3, T, H, W]``; a 4-D tensor is one clip without its batch axis (``CTHW`` / ``TCHW``)."""
    shape = tuple(video.shape)
    problem = f"media tensor must contain RGB video in BCTHW/CTHW or BTCHW/TCHW layout, got {shape}"
    if video.ndim not in (4, 5):
        raise ValueError(problem)
    if layout not in ("BCTHW", "BTCHW"):
        raise ValueError(f"unsupported media layout: {layout!r}")
    if video.ndim == 4:
        video = video.unsqueeze(0)
    if layout == "BTCHW":
        video = video.permute(0, 2, 1, 3, 4)
    if video.shape[1] != 3:
        raise ValueError(problem)
    return video


def _to_uint8(video: Tensor, float_range: str, chunk: int) -> Tensor:
    """``[3, T, H, W]`` -> CPU uint8 ``[T, H, W, 3]``, converted ``chunk`` frames at a time so that
    a long clip never holds a second full-size copy on the device."""
    c, t, h, w = video.shape
    if c != 3:
        raise ValueError(f"media tensor must have three RGB channels, got {c}")
    if chunk <= 0:
        raise ValueError("frame_chunk_size must be positive")
    if video.dtype != torch.uint8 and not video.is_floating_point():
        raise TypeError(f"media tensor must be floating point or uint8, got {video.dtype}")
    if float_range not in ("minus_one_one", "zero_one"):
        raise ValueError(f"unsupported floating-point range: {float_range!r}")
    out = torch.empty((t, h, w, 3), dtype=torch.uint8)
    for lo in range(0, t, chunk):
        part = video[:, lo:lo + chunk].detach()
        if part.dtype != torch.uint8:
            part = part.float()
            part = (part + 1.0) * 127.5 if float_range == "minus_one_one" else part * 255.0
            part = part.round().clamp_(0, 255).to(torch.uint8)
        out[lo:lo + part.shape[1]].copy_(part.permute(1, 2, 3, 0).cpu())
    return out


def _clips_uint8(value: Tensor, layout: str, float_range: str, frame_chunk_size: int) -> list[Tensor]:
    """One CPU uint8 ``[T, H, W, 3]`` clip per sample (the layout the encoders take)."""
    return [_to_uint8(v, float_range, frame_chunk_size) for v in _canonical(value, layout)]


def video_batch_to_cpu_uint8(value: Tensor, *, layout: str = "BCTHW",
                             float_range: str = "minus_one_one", frame_chunk_size: int = 8) -> Tensor:
    """A media batch as one CPU uint8 tensor ``[B, C, T, H, W]``, converted a few frames at a
    time (reference ``wm/infra/callbacks/media.py:84-100``)."""
    clips = _clips_uint8(value, layout, float_range, frame_chunk_size)
    return torch.stack([clip.permute(3, 0, 1, 2) for clip in clips])


def _resize(pixels: Tensor, size: tuple[int, int], chunk: int) -> Tensor:
    if tuple(pixels.shape[1:3]) == tuple(size):
        return pixels
    out = torch.empty((pixels.shape[0], *size, 3), dtype=torch.uint8)
    for lo in range(0, pixels.shape[0], chunk):
        part = pixels[lo:lo + chunk].permute(0, 3, 1, 2).float()
        part = F.interpolate(part, size=size, mode="bilinear", align_corners=False)
        out[lo:lo + part.shape[0]].copy_(part.round().clamp_(0, 255).to(torch.uint8).permute(0, 2, 3, 1))
    return out


class ImageVideoArtifactWriter:
    def __init__(self, *, layout: str = "BCTHW", float_range: str = "minus_one_one", fps: int = 16,
                 frame_chunk_size: int = 8, image_format: str = "jpg", image_quality: int = 90,
                 video_quality: int = 5, grid_layout: Sequence[Any] | None = None,
                 grid_condition_keys: Sequence[Any] | None = None, grid_reference_key: Any | None = None,
                 grid_name: str = "grid", save_individual_artifacts: bool = True,
                 async_write: bool = False) -> None:
        self.layout, self.float_range = layout, float_range
        self.fps, self.frame_chunk_size = int(fps), int(frame_chunk_size)
        self.image_format, self.image_quality = image_format, int(image_quality)
        self.video_quality = int(video_quality)
        self.grid_layout = None if grid_layout is None else tuple(grid_layout)
        if self.grid_layout is not None:
            if len(self.grid_layout) not in (3, 4):
                raise ValueError("video grid layout must contain three or four artifact keys")
            if len(set(self.grid_layout)) != len(self.grid_layout):
                raise ValueError("video grid layout keys must be unique")
            default = self.grid_layout[: 1 if len(self.grid_layout) == 3 else 2]
            self.grid_condition_keys = frozenset(default if grid_condition_keys is None
                                                 else grid_condition_keys)
            if not self.grid_condition_keys.issubset(self.grid_layout):
                raise ValueError("video grid condition keys must belong to the grid layout")
            self.grid_reference_key = self.grid_layout[-1] if grid_reference_key is None \
                else grid_reference_key
            if self.grid_reference_key not in self.grid_layout:
                raise ValueError("video grid reference key must belong to the grid layout")
        else:
            self.grid_condition_keys, self.grid_reference_key = frozenset(), None
        self.grid_name = str(grid_name)
        self.save_individual_artifacts = bool(save_individual_artifacts)
        self.async_write = bool(async_write)
        self._failed = False
        self._worker: Thread | None = None

    # -------------------------------------------------------------------- building
    def _grids(self, artifacts: Mapping[Any, Any]) -> Iterator[tuple[int, int, Tensor]]:
        videos = {}
        for key in self.grid_layout:
            if not torch.is_tensor(artifacts[key]):
                raise TypeError(f"media artifact {key!r} is not a tensor")
            videos[key] = _canonical(artifacts[key], self.layout)
        sizes = {int(v.shape[0]) for v in videos.values()}
        if len(sizes) != 1:
            raise ValueError("video grid artifacts must share one batch size")
        frames = min(int(v.shape[2]) for v in videos.values())
        if frames <= 0:
            raise ValueError("video grid artifacts must contain at least one frame")
        h, w = (int(s) for s in videos[self.grid_reference_key].shape[-2:])
        for key, v in videos.items():
            if key not in self.grid_condition_keys and tuple(v.shape[-2:]) != (h, w):
                raise ValueError("non-condition video grid artifacts must match the reference "
                                 f"spatial size; {key!r} has {tuple(v.shape[-2:])}, reference "
                                 f"{self.grid_reference_key!r} has {(h, w)}")
        rows, cols = (1, 3) if len(self.grid_layout) == 3 else (2, 2)
        batch = next(iter(sizes))
        for b in range(batch):
            grid = torch.zeros((frames, rows * h, cols * w, 3), dtype=torch.uint8)
            for i, key in enumerate(self.grid_layout):
                pixels = _to_uint8(videos[key][b, :, :frames], self.float_range, self.frame_chunk_size)
                if key in self.grid_condition_keys:
                    pixels = _resize(pixels, (h, w), self.frame_chunk_size)
                r, c = divmod(i, cols)
                grid[:, r * h:(r + 1) * h, c * w:(c + 1) * w].copy_(pixels)
            yield b, batch, grid

    def _artifacts(self, value: Any) -> Iterator[tuple[str, int, int, Tensor]]:
        """``(name, index in batch, batch size, uint8 [T, H, W, 3])`` of everything to be written:
        the grid first when all its panels are present, then (unless a grid was built and single
        artifacts are switched off) every entry by sorted key.  Names are made file-safe and kept
        distinct; an entry that is not a tensor is an error (reference
        ``wm/infra/callbacks/media.py:248-317``)."""
        named = {"sample": value} if torch.is_tensor(value) else value
        if not isinstance(named, Mapping):
            raise TypeError("image/video sample must be a tensor or a mapping of tensors")
        taken: set[str] = set()
        with_grid = self.grid_layout is not None and all(key in named for key in self.grid_layout)
        if with_grid:
            title = _safe(self.grid_name)
            taken.add(title)
            for b, batch, grid in self._grids(named):
                yield title, b, batch, grid
            if not self.save_individual_artifacts:
                return
        for key in sorted(named, key=str):
            tensor = named[key]
            if not torch.is_tensor(tensor):
                raise TypeError(f"media artifact {key!r} is not a tensor")
            stem = name = _safe(key)
            attempt = 2
            while name in taken:
                name, attempt = f"{stem}_{attempt}", attempt + 1
            taken.add(name)
            clips = _clips_uint8(tensor, self.layout, self.float_range, self.frame_chunk_size)
            for b, pixels in enumerate(clips):
                yield name, b, len(clips), pixels

    # --------------------------------------------------------------------- writing
    def _publish(self, jobs: Sequence[tuple[Tensor, str]]) -> None:
        for pixels, destination in jobs:
            if pixels.shape[0] == 1:
                options = {"quality": self.image_quality} if self.image_format in ("jpg", "jpeg") else {}
                fmt = "JPEG" if self.image_format in ("jpg", "jpeg") else self.image_format.upper()
                buffer = io.encode_image(pixels[0].numpy(), file_format=fmt, **options)
            else:
                buffer = io.encode_video(pixels.numpy(), fps=self.fps, quality=self.video_quality)
            io.atomic_put(buffer, destination)

    def _publish_in_thread(self, jobs) -> None:
        try:
            self._publish(jobs)
        except Exception as error:
            if not self._failed:
                self._failed = True
                log.warning("Disabling asynchronous media writes after failure: "
                            f"{type(error).__name__}: {error}")

    def _join(self) -> None:
        if self._worker is not None:
            self._worker.join()
            self._worker = None

    def write(self, value: Any, *, output_dir: str, split: str, iteration: int, rank: int,
              sample_batch_index: int = 0) -> None:
        del split
        if self._failed:
            return
        if self.async_write:
            self._join()
            if self._failed:
                return
        jobs = []
        for name, b, batch, pixels in self._artifacts(value):
            extension = self.image_format if pixels.shape[0] == 1 else "mp4"
            filename = media_artifact_filename(
                artifact_name=name, iteration=iteration, rank=rank,
                sample_batch_index=sample_batch_index, extension=extension,
                batch_index=b if batch > 1 else None)
            jobs.append((pixels, io.join_path(str(output_dir), filename)))
        if not jobs:
            return
        if not self.async_write:
            self._publish(jobs)
            return
        self._worker = Thread(target=self._publish_in_thread, args=(jobs,), name="media-writer")
        self._worker.start()

    def close(self) -> None:
        self._join()
