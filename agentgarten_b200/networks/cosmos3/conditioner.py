"""Raw batch → latents and conditions.

Raw batch: ``video [B,T,3,H,W]`` (uint8 or [-1,1]), ``depth [B,T,1,H,W]`` metric,
``depth_scale [B]``, ``normal [B,T,3,H,W]`` unit vectors, ``caption`` (or
``text_input_ids``), ``fps [B]``, optional ``sample_id [B]``.  A precomputed ``latent``
replaces ``video``; ``depth_latent`` + ``normal_latent`` (both or neither) replace
``depth``/``normal``.  With all four cached keys present, neither the VAE nor the
tokenizer is touched — the path synthetic benchmarks use.

``condition()`` runs the frozen text tower and packages its per-layer K/V with the
geometry latents and the frame rate.

The work is split over three small collaborators: :class:`_Prompts` turns captions into padded
token rows (caption suffix with duration, frame rate and resolution, chat template, the
negative prompt file), :class:`_Geometry` turns metric depth and normals into noised VAE
latents, and the conditioner itself owns the frozen text tower and assembles conditions.

Parity: reference ``wm/networks/cosmos3/conditioner.py:44-370`` (constructor keywords, batch
keys in and out, seeds of the validation noise).
"""

from __future__ import annotations

import json
from collections.abc import Mapping, Sequence
from pathlib import Path
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

from .layers import Cosmos3Config
from .network import Cosmos3Condition, Cosmos3TextEncoder

__all__ = ["COSMOS3_EMPTY_PROMPT_IDS", "Cosmos3Conditioner"]

# Chat template around an empty user message: used for text dropout and as the default
# negative prompt.
from agentgarten_b200.networks.cosmos3 import COSMOS3_EMPTY_PROMPT_IDS  # noqa: E402
# Validation geometry noise is seeded per modality and sample id, so it is identical across
# guidance arms, solver steps, evaluation rounds and batchings.
_EVAL_NOISE_SEED = {"depth": 23_071_996 + 0x1D3E7A11, "normal": 23_071_996 + 0x4A6F2C35}


class _Prompts:
    """Captions → token ids.  The tokenizer is loaded on first use."""

    def __init__(self, tokenizer_path: str | None, negative_prompt_path: str | None,
                 max_tokens: int, default_fps: float) -> None:
        self.tokenizer_path, self.negative_prompt_path = tokenizer_path, negative_prompt_path
        self.max_tokens, self.default_fps = int(max_tokens), float(default_fps)
        self.tokenizer: Any = None
        self.negative_text: str | None = None

    def _rows(self, prompts: Sequence[str]) -> tuple[torch.Tensor, torch.Tensor]:
        """Chat-templated ids of every prompt, right-padded with zeros, and the validity mask."""
        if self.tokenizer is None:
            if self.tokenizer_path is None:
                raise ValueError("captions need Cosmos3Conditioner(tokenizer_path=...)")
            from transformers import AutoTokenizer

            self.tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_path, local_files_only=True)
        encoded = []
        for prompt in prompts:
            ids = self.tokenizer.apply_chat_template([{"role": "user", "content": prompt}], tokenize=True,
                                                     add_generation_prompt=True, add_vision_id=False,
                                                     return_dict=False)
            ids = ids.flatten().tolist() if torch.is_tensor(ids) else list(ids)
            encoded.append(ids[: self.max_tokens])
        longest = max(len(ids) for ids in encoded)
        table = torch.zeros(len(encoded), longest, dtype=torch.long)
        valid = torch.zeros(len(encoded), longest, dtype=torch.bool)
        for row, ids in enumerate(encoded):
            table[row, : len(ids)] = torch.tensor(ids)
            valid[row, : len(ids)] = True
        return table, valid

    def _negative(self) -> str:
        if self.negative_text is None:
            payload = json.loads(Path(self.negative_prompt_path).read_text())
            self.negative_text = json.dumps(payload).rstrip(".") + "."
        return self.negative_text

    def fill(self, batch: dict[str, Any], pixel_shape: Sequence[int], device: torch.device, *,
             training: bool) -> None:
        """Replace ``caption`` by ``text_input_ids`` / ``text_attention_mask`` (and, outside
        training, the negative prompt's rows) unless ids are already present."""
        if "caption" not in batch or "text_input_ids" in batch:
            return
        samples, _, frames, height, width = pixel_shape
        rates = torch.as_tensor(batch.get("fps", self.default_fps)).float().reshape(-1)
        rates = [float(r) for r in (rates.expand(samples) if rates.numel() == 1 else rates)]
        tails = [f" The video is {frames / rate:.1f} seconds long and is of {rate:.0f} FPS. "
                 f"This video is of {height}x{width} resolution." for rate in rates]
        captions = batch.pop("caption")
        ids, valid = self._rows([text.strip() + tail for text, tail in zip(captions, tails)])
        batch["text_input_ids"], batch["text_attention_mask"] = ids.to(device), valid.to(device)
        if training or self.negative_prompt_path is None:
            return
        ids, valid = self._rows([self._negative() + tail for tail in tails])
        batch["negative_text_input_ids"], batch["negative_text_attention_mask"] = ids.to(device), valid.to(device)


class _Geometry:
    """Metric depth + unit normals → control videos → VAE latents → noised latents."""

    def __init__(self, codec: Any, augmentation: Any, noise_sigma: float) -> None:
        self.codec, self.augmentation, self.noise_sigma = codec, augmentation, float(noise_sigma)

    def videos(self, batch: dict[str, Any], *, training: bool) -> dict[str, torch.Tensor]:
        from . import geometry as G

        options = self.augmentation
        depth = _channels_first(batch["depth"], channels=1).float()
        batch.setdefault("depth_scale", torch.ones(depth.shape[0]))
        scale = G.depth_scale(batch, training=training, batch_size=depth.shape[0])
        controls = {"depth": G.colorize_depth(depth, scale),
                    "normal": G.prepare_normal(_channels_first(batch["normal"], channels=3))}
        controls = G.downsample_geometry(controls, factor=options.geometry_spatial_downsample)
        controls = G.augment_geometry(controls, data_batch=batch, training=training, config=options)
        controls = G.stretch_geometry(controls, training=training, divisor=options.geometry_stretch_divisor)
        controls["depth"] = controls["depth"] * 2.0 - 1.0  # colours in [0, 1] → the VAE's [-1, 1]
        return {name: video.to(self.codec.dtype).contiguous() for name, video in controls.items()}

    def latents(self, videos: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """Depth and normal of one sample go through the VAE together, as a batch of two."""
        encoded: dict[str, list[torch.Tensor]] = {"depth": [], "normal": []}
        for sample in range(videos["depth"].shape[0]):
            both = torch.cat((videos["depth"][sample:sample + 1], videos["normal"][sample:sample + 1]))
            depth, normal = self.codec.encode(both).float().split(1)
            encoded["depth"].append(depth)
            encoded["normal"].append(normal)
        return {name: torch.cat(parts) for name, parts in encoded.items()}

    def noised(self, latent: torch.Tensor, modality: str, sample_ids: Sequence[int], *,
               training: bool) -> torch.Tensor:
        """Blend with Gaussian noise: fresh in training, seeded by (modality, sample id) else."""
        sigma = self.noise_sigma
        if sigma == 0.0:
            return latent
        if training:
            noise = torch.randn(latent.shape, device=latent.device)
        else:
            noise = torch.stack([
                torch.randn(latent.shape[1:], device=latent.device,
                            generator=torch.Generator(device=latent.device).manual_seed(
                                _EVAL_NOISE_SEED[modality] + int(sample_id)))
                for sample_id in sample_ids])
        return latent * (1.0 - sigma) + noise * sigma


class Cosmos3Conditioner(nn.Module):
    def __init__(self, *, config: Cosmos3Config, codec: Any = None,
                 geometry_augmentation: Any = None, geometry_noise_sigma: float = 0.4,
                 empty_prompt_ids: Sequence[int] = COSMOS3_EMPTY_PROMPT_IDS,
                 default_fps: float = 16.0, tokenizer_path: str | None = None,
                 negative_prompt_path: str | None = None, max_text_tokens: int = 512,
                 init_device: str = "meta") -> None:
        super().__init__()
        if not 0.0 <= geometry_noise_sigma <= 1.0:
            raise ValueError(f"geometry_noise_sigma must be in [0, 1], got {geometry_noise_sigma}")
        from . import _as_config

        with torch.device(init_device):
            self.text_encoder = Cosmos3TextEncoder(_as_config(config))
        self.text_encoder.requires_grad_(False)
        self.codec = codec  # a plain attribute: nothing of it is trained or checkpointed
        if geometry_augmentation is None:
            from .geometry import GeometryAugmentationConfig

            geometry_augmentation = GeometryAugmentationConfig()
        self.geometry_augmentation = geometry_augmentation
        self.geometry_noise_sigma = float(geometry_noise_sigma)
        self.empty_prompt_ids = tuple(int(token) for token in empty_prompt_ids)
        self.default_fps = float(default_fps)
        self.tokenizer_path, self.negative_prompt_path = tokenizer_path, negative_prompt_path
        self.max_text_tokens = int(max_text_tokens)
        self._prompts = _Prompts(tokenizer_path, negative_prompt_path, self.max_text_tokens, self.default_fps)
        # The text tower's output can be memoised by prompt: prompts repeat across guidance arms
        # and denoising steps of a sampling run.  Off unless a caller switches it on.
        self.cache_text_contexts = False
        self._text_cache: dict[bytes, Any] = {}

    def train(self, mode: bool = True) -> "Cosmos3Conditioner":
        super().train(mode)
        self.text_encoder.eval()  # frozen: never in training mode
        return self

    def _geometry(self) -> _Geometry:
        return _Geometry(self.codec, self.geometry_augmentation, self.geometry_noise_sigma)

    # ---------------------------------------------------------------------- encode
    def _pixel_shape(self, latent: torch.Tensor) -> tuple[int, ...]:
        """Shape of the video a cached latent stands for (4 n + 1 frames of 16 h x 16 w)."""
        samples, channels, frames, height, width = latent.shape
        if self.codec is None:
            return (samples, channels, 4 * (frames - 1) + 1, 16 * height, 16 * width)
        factor = self.codec.spatial_compression_factor
        return (samples, channels, self.codec.pixel_frames(frames), height * factor, width * factor)

    @torch.no_grad()
    def encode(self, batch: Mapping[str, Any], *, training: bool) -> dict[str, Any]:
        out = dict(batch)
        # 1. the clip itself
        if "latent" in out:
            out.pop("video", None)
            pixel_shape = self._pixel_shape(out["latent"])
        else:
            video = _to_unit_range(out.pop("video"))
            pixel_shape = tuple(video.shape)
            out["latent"] = torch.cat([self.codec.encode(video[i:i + 1]) for i in range(video.shape[0])]).float()
        samples, device = out["latent"].shape[0], out["latent"].device
        # 2. the prompt
        self._prompts.fill(out, pixel_shape, self.text_encoder.embed_tokens.weight.device, training=training)
        # 3. the controls
        have = [key in out for key in ("depth_latent", "normal_latent")]
        if have[0] != have[1]:
            raise ValueError("cache both depth_latent and normal_latent, or neither")
        if not have[0]:
            geometry = self._geometry()
            videos = geometry.videos(out, training=training)
            if not training:  # panels for the sample grids
                out["depth_video"], out["normal_video"] = videos["depth"], videos["normal"]
            identifiers = out.get("sample_id")
            identifiers = list(range(samples)) if identifiers is None \
                else torch.as_tensor(identifiers).reshape(-1).tolist()
            for modality, latent in geometry.latents(videos).items():
                out[f"{modality}_latent"] = geometry.noised(latent, modality, identifiers, training=training)
        out.pop("depth", None)
        out.pop("normal", None)
        # 4. the frame rate
        out.setdefault("fps", torch.full((samples,), self.default_fps, device=device))
        return out

    # ------------------------------------------------------------------- condition
    def _blank_prompt(self, samples: int, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
        ids = torch.tensor(self.empty_prompt_ids, device=device).expand(samples, -1)
        return ids, torch.ones_like(ids, dtype=torch.bool)

    def _prompt_rows(self, batch: Mapping[str, Any], negative: bool) -> tuple[torch.Tensor, torch.Tensor]:
        key = "negative_text_input_ids" if negative else "text_input_ids"
        ids = batch.get(key)
        if ids is None:
            if negative:  # no negative prompt configured: the empty chat message
                return self._blank_prompt(batch["latent"].shape[0], batch["latent"].device)
            raise KeyError("batch has neither caption nor text_input_ids")
        valid = batch.get(key.replace("input_ids", "attention_mask"))
        return ids, (torch.ones_like(ids, dtype=torch.bool) if valid is None else valid.bool())

    def _context(self, ids: torch.Tensor, valid: torch.Tensor):
        if not self.cache_text_contexts:
            return self.text_encoder(ids, valid)
        key = (ids * valid).cpu().numpy().tobytes() + valid.cpu().numpy().tobytes()
        if key not in self._text_cache:
            if len(self._text_cache) > 16:
                self._text_cache.clear()
            self._text_cache[key] = self.text_encoder(ids, valid)
        return self._text_cache[key]

    @torch.no_grad()
    def condition(self, batch: Mapping[str, Any], *, negative: bool = False,
                  drop: torch.Tensor | None = None) -> Cosmos3Condition:
        """``drop`` [B] bool: those rows get the empty prompt (text dropout of training)."""
        ids, valid = self._prompt_rows(batch, negative)
        if drop is not None and not negative:
            ids, valid = _choose_rows(drop, self._blank_prompt(ids.shape[0], ids.device), (ids, valid))
        rate = torch.as_tensor(batch["fps"], dtype=torch.float32).reshape(-1)
        return Cosmos3Condition(text=self._context(ids, valid), depth=batch["depth_latent"],
                                normal=batch["normal_latent"], fps=rate)

    # --------------------------------------------------------------------- outputs
    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        return self.codec.decode(latent).float()

    def visuals(self, batch: Mapping[str, Any]) -> dict[str, torch.Tensor]:
        panels = {}
        for modality in ("depth", "normal"):
            video = batch.get(f"{modality}_video")
            if video is not None:
                panels[modality] = video.float()
        return panels


def _channels_first(value: torch.Tensor, *, channels: int) -> torch.Tensor:
    """[B, T, C, H, W] → [B, C, T, H, W], checking the channel count."""
    if value.ndim != 5 or value.shape[2] != channels:
        raise ValueError(f"expected [B, T, {channels}, H, W], got {tuple(value.shape)}")
    return value.permute(0, 2, 1, 3, 4)


def _to_unit_range(video: torch.Tensor) -> torch.Tensor:
    """uint8 frames to [-1, 1]; float frames are taken to be in that range already."""
    frames = _channels_first(video, channels=3)
    return frames.float() / 127.5 - 1.0 if frames.dtype == torch.uint8 else frames.float()


def _choose_rows(pick_first: torch.Tensor, first, second):
    """Row-wise choice between two (ids, mask) pairs of possibly different widths."""
    width = max(first[0].shape[1], second[0].shape[1])

    def widened(pair):
        ids, valid = pair
        room = width - ids.shape[1]
        return F.pad(ids, (0, room)), F.pad(valid, (0, room), value=False)

    (ids_a, valid_a), (ids_b, valid_b) = widened(first), widened(second)
    chooser = pick_first.to(device=ids_b.device, dtype=torch.bool)[:, None]
    return torch.where(chooser, ids_a, ids_b), torch.where(chooser, valid_a, valid_b)
