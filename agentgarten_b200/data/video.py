"""Datasets: JSONL manifests of real clips, and seeded synthetic clips / latents.

A manifest row is ``{"video": path, "depth": path.npy, "normal": path.(mp4|npy),
"caption": str, "depth_scale": float}`` with paths relative to the manifest.  Samples are
checked strictly (frame count, resolution, finite values, non-negative depth).

Parity: reference ``wm/data/video.py:28-149``; ``SyntheticLatentDataset`` (cached latents,
the form the benchmarks use) is an addition.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any

import numpy as np
import torch
from torch.utils.data import Dataset

__all__ = ["ManifestVideoDataset", "SyntheticLatentDataset", "SyntheticVideoDataset"]


def _read_video(path: Path) -> torch.Tensor:
    """All frames as uint8 ``[T, 3, H, W]``.

    ``.npy`` files hold the frames directly (``[T, H, W, 3]`` or ``[T, 3, H, W]`` uint8).
    Encoded videos are decoded by torchcodec when it is installed, else by OpenCV.
    """
    if path.suffix == ".npy":
        frames = torch.from_numpy(np.load(path))
        if frames.dtype != torch.uint8 or frames.ndim != 4:
            raise ValueError(f"{path}: expected uint8 frames [T, H, W, 3] or [T, 3, H, W]")
        return frames if frames.shape[1] == 3 else frames.permute(0, 3, 1, 2).contiguous()
    try:
        from torchcodec.decoders import VideoDecoder
    except ImportError:
        VideoDecoder = None
    if VideoDecoder is not None:
        decoder = VideoDecoder(str(path))
        return decoder.get_frames_in_range(0, len(decoder)).data
    try:
        import cv2
    except ImportError as error:
        raise ImportError("reading encoded videos needs torchcodec or opencv") from error
    capture = cv2.VideoCapture(str(path))
    frames = []
    try:
        while True:
            ok, frame = capture.read()
            if not ok:
                break
            frames.append(torch.from_numpy(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB)))
    finally:
        capture.release()
    if not frames:
        raise ValueError(f"{path}: no frames could be decoded")
    return torch.stack(frames).permute(0, 3, 1, 2).contiguous()


class ManifestVideoDataset(Dataset):
    def __init__(self, manifest: str, *, num_frames: int, height: int, width: int,
                 fps: float = 16.0) -> None:
        self.path = Path(manifest)
        text = self.path.read_text()
        self.rows = [json.loads(line) for line in text.splitlines() if line.strip()]
        if not self.rows:
            raise ValueError(f"manifest {manifest} is empty")
        self.digest = hashlib.sha256(text.encode()).hexdigest()
        self.num_frames, self.height, self.width = int(num_frames), int(height), int(width)
        self.fps = float(fps)

    def __len__(self) -> int:
        return len(self.rows)

    def resume_signature(self) -> dict[str, Any]:
        return {"manifest": self.digest, "num_frames": self.num_frames, "height": self.height,
                "width": self.width, "fps": self.fps}

    def _resolve(self, value: str) -> Path:
        p = Path(value)
        return p if p.is_absolute() else self.path.parent / p

    def _checked(self, path: Path, value: torch.Tensor, tail: tuple) -> torch.Tensor:
        want = (self.num_frames, *tail)
        if tuple(value.shape) != want:
            raise ValueError(f"{path}: expected {want} (frames, ...), got {tuple(value.shape)}")
        if value.is_floating_point() and not torch.isfinite(value).all():
            raise ValueError(f"{path}: contains non-finite values")
        return value

    def __getitem__(self, index: int) -> dict[str, Any]:
        row = self.rows[index]
        hw = (self.height, self.width)
        video_path = self._resolve(row["video"])
        video = self._checked(video_path, _read_video(video_path), (3, *hw))
        depth_path = self._resolve(row["depth"])
        depth = self._checked(depth_path, torch.from_numpy(np.load(depth_path)).float(), hw)
        if (depth < 0).any():
            raise ValueError(f"{depth_path}: depth must be non-negative")
        normal_path = self._resolve(row["normal"])
        if normal_path.suffix == ".npy":
            normal = torch.from_numpy(np.load(normal_path)).float()
            normal = self._checked(normal_path, normal, (*hw, 3)).permute(0, 3, 1, 2)
        else:
            normal = self._checked(normal_path, _read_video(normal_path).float() / 127.5 - 1.0, (3, *hw))
        normal = normal / normal.norm(dim=1, keepdim=True).clamp_min(1e-6)
        return {"video": video, "depth": depth[:, None], "normal": normal,
                "caption": str(row.get("caption", "")), "fps": self.fps,
                "depth_scale": float(row.get("depth_scale", 1.0)), "sample_id": index}


class SyntheticVideoDataset(Dataset):
    """Seeded random pixel clips with depth and unit normals."""

    def __init__(self, *, length: int, num_frames: int, height: int, width: int,
                 fps: float = 16.0) -> None:
        self.length, self.num_frames = int(length), int(num_frames)
        self.height, self.width, self.fps = int(height), int(width), float(fps)

    def __len__(self) -> int:
        return self.length

    def __getitem__(self, index: int) -> dict[str, Any]:
        g = torch.Generator().manual_seed(index)
        t, h, w = self.num_frames, self.height, self.width
        normal = torch.randn(t, 3, h, w, generator=g)
        return {"video": torch.randint(0, 256, (t, 3, h, w), generator=g, dtype=torch.uint8),
                "depth": 1.0 + 9.0 * torch.rand(t, 1, h, w, generator=g),
                "normal": normal / normal.norm(dim=1, keepdim=True),
                "caption": f"synthetic clip {index}", "fps": self.fps, "depth_scale": 1.0,
                "sample_id": index}


class SyntheticLatentDataset(Dataset):
    """Seeded cached-latent samples: ``latent``, ``depth_latent``, ``normal_latent`` ~ N(0,1)
    and random prompt ids, which bypass the VAE and the tokenizer in the conditioner."""

    def __init__(self, *, length: int, latent_frames: int, latent_height: int, latent_width: int,
                 channels: int = 48, text_tokens: int = 512, vocab_size: int = 151936,
                 fps: float = 16.0, geometry_height: int | None = None,
                 geometry_width: int | None = None) -> None:
        self.length = int(length)
        self.shape = (int(channels), int(latent_frames), int(latent_height), int(latent_width))
        self.geometry_shape = (int(channels), int(latent_frames), int(geometry_height or latent_height),
                               int(geometry_width or latent_width))
        self.text_tokens, self.vocab_size, self.fps = int(text_tokens), int(vocab_size), float(fps)

    def __len__(self) -> int:
        return self.length

    def resume_signature(self) -> dict[str, Any]:
        return {"shape": list(self.shape), "geometry": list(self.geometry_shape),
                "text_tokens": self.text_tokens}

    def __getitem__(self, index: int) -> dict[str, Any]:
        g = torch.Generator().manual_seed(index)
        return {"latent": torch.randn(self.shape, generator=g),
                "depth_latent": torch.randn(self.geometry_shape, generator=g),
                "normal_latent": torch.randn(self.geometry_shape, generator=g),
                "text_input_ids": torch.randint(3, self.vocab_size, (self.text_tokens,), generator=g),
                "fps": self.fps, "sample_id": index}
