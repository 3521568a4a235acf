"""Raw batch → latents and conditions.

Raw batch: ``video [B,T,3,H,W]`` (uint8 or [-1,1]), ``depth [B,T,1,H,W]`` metric,
``depth_scale [B]``, ``normal [B,T,3,H,W]`` unit vectors, ``caption`` (or
``text_input_ids``), ``fps [B]``, optional ``sample_id [B]``.  A precomputed ``latent``
replaces ``video``; ``depth_latent`` + ``normal_latent`` (both or neither) replace
``depth``/``normal``.  With all four cached keys present, neither the VAE nor the
tokenizer is touched — the path synthetic benchmarks use.

``condition()`` runs the frozen text tower and packages its per-layer K/V with the
geometry latents and the frame rate.

Parity: reference ``wm/networks/cosmos3/conditioner.py:44-370``.
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
        self.codec = codec  # plain attribute: no trainable or checkpointed state
        if geometry_augmentation is None:
            from .geometry import GeometryAugmentationConfig

            geometry_augmentation = GeometryAugmentationConfig()
        self.geometry_augmentation = geometry_augmentation
        self.geometry_noise_sigma = float(geometry_noise_sigma)
        self.empty_prompt_ids = tuple(int(t) for t in empty_prompt_ids)
        self.default_fps = float(default_fps)
        self.tokenizer_path = tokenizer_path
        self.negative_prompt_path = negative_prompt_path
        self.max_text_tokens = int(max_text_tokens)
        self._tokenizer: Any = None
        self._negative_prompt: str | None = None
        # Optional memo of the text tower output keyed by the prompt ids: prompts repeat
        # across guidance arms and denoising steps.
        self._text_cache: dict[bytes, Any] = {}
        self.cache_text_contexts = False

    def train(self, mode: bool = True) -> "Cosmos3Conditioner":
        super().train(mode)
        self.text_encoder.eval()
        return self

    # ---------------------------------------------------------------------- encode
    @torch.no_grad()
    def encode(self, batch: Mapping[str, Any], *, training: bool) -> dict[str, Any]:
        out = dict(batch)
        if "latent" in out:
            out.pop("video", None)
            shape = self._pixel_shape(out["latent"])
        else:
            video = _pixels(out.pop("video"))
            shape = tuple(video.shape)
            out["latent"] = self._encode_each(video)
        self._tokenize_prompts(out, shape, training=training)
        cached = ("depth_latent" in out) + ("normal_latent" in out)
        if cached == 1:
            raise ValueError("cache both depth_latent and normal_latent, or neither")
        if not cached:
            pixels = self._geometry_pixels(out, training=training)
            if not training:
                out["depth_video"], out["normal_video"] = pixels["depth"], pixels["normal"]
            ids = out.get("sample_id")
            ids = list(range(out["latent"].shape[0])) if ids is None \
                else torch.as_tensor(ids).reshape(-1).tolist()
            for name, latent in self._encode_geometry(pixels).items():
                out[f"{name}_latent"] = self._geometry_noise(
                    latent, name, training=training, sample_ids=ids)
        out.pop("depth", None)
        out.pop("normal", None)
        if "fps" not in out:
            out["fps"] = torch.full((out["latent"].shape[0],), self.default_fps,
                                    device=out["latent"].device)
        return out

    def _pixel_shape(self, latent: torch.Tensor) -> tuple[int, ...]:
        b, c, t, h, w = latent.shape
        if self.codec is None:
            return (b, c, 4 * (t - 1) + 1, h * 16, w * 16)
        f = self.codec.spatial_compression_factor
        return (b, c, self.codec.pixel_frames(t), h * f, w * f)

    def _tokenize_prompts(self, batch: dict[str, Any], shape: Sequence[int], *,
                          training: bool) -> None:
        if "caption" not in batch or "text_input_ids" in batch:
            return
        _, _, frames, height, width = shape
        fps = torch.as_tensor(batch.get("fps", self.default_fps)).float().reshape(-1)
        fps = fps.expand(shape[0]) if fps.numel() == 1 else fps

        def suffix(i: int) -> str:
            rate = float(fps[i])
            return (f" The video is {frames / rate:.1f} seconds long and is of {rate:.0f} FPS. "
                    f"This video is of {height}x{width} resolution.")

        captions = batch.pop("caption")
        prompts = [c.strip() + suffix(i) for i, c in enumerate(captions)]
        batch["text_input_ids"], batch["text_attention_mask"] = self._tokenize(prompts)
        if not training and self.negative_prompt_path is not None:
            if self._negative_prompt is None:
                payload = json.loads(Path(self.negative_prompt_path).read_text())
                self._negative_prompt = json.dumps(payload).rstrip(".") + "."
            rows = [self._negative_prompt + suffix(i) for i in range(len(prompts))]
            ids, mask = self._tokenize(rows)
            batch["negative_text_input_ids"], batch["negative_text_attention_mask"] = ids, mask

    def _tokenize(self, prompts: Sequence[str]) -> tuple[torch.Tensor, torch.Tensor]:
        if self._tokenizer is None:
            if self.tokenizer_path is None:
                raise ValueError("captions need Cosmos3Conditioner(tokenizer_path=...)")
            from transformers import AutoTokenizer

            self._tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_path,
                                                            local_files_only=True)
        rows = []
        for prompt in prompts:
            ids = self._tokenizer.apply_chat_template(
                [{"role": "user", "content": prompt}], tokenize=True,
                add_generation_prompt=True, return_dict=False)
            ids = ids.flatten().tolist() if torch.is_tensor(ids) else list(ids)
            rows.append(torch.tensor(ids[: self.max_text_tokens]))
        width = max(r.numel() for r in rows)
        ids = torch.zeros(len(rows), width, dtype=torch.long)
        mask = torch.zeros(len(rows), width, dtype=torch.bool)
        for i, r in enumerate(rows):
            ids[i, : r.numel()] = r
            mask[i, : r.numel()] = True
        device = self.text_encoder.embed_tokens.weight.device
        return ids.to(device), mask.to(device)

    def _encode_each(self, pixels: torch.Tensor) -> torch.Tensor:
        return torch.cat([self.codec.encode(pixels[i:i + 1]) for i in range(pixels.shape[0])]).float()

    def _geometry_pixels(self, batch: dict[str, Any], *, training: bool) -> dict[str, torch.Tensor]:
        from . import geometry as G

        config = self.geometry_augmentation
        depth = _canonical(batch["depth"], channels=1).float()
        batch.setdefault("depth_scale", torch.ones(depth.shape[0]))
        scale = G.depth_scale(batch, training=training, batch_size=depth.shape[0])
        videos = G.downsample_geometry(
            {"depth": G.colorize_depth(depth, scale),
             "normal": G.prepare_normal(_canonical(batch["normal"], channels=3))},
            factor=config.geometry_spatial_downsample)
        videos = G.augment_geometry(videos, data_batch=batch, training=training, config=config)
        videos = G.stretch_geometry(videos, training=training,
                                    divisor=config.geometry_stretch_divisor)
        videos["depth"] = videos["depth"] * 2.0 - 1.0  # [0,1] colours → VAE range
        return {k: v.to(self.codec.dtype).contiguous() for k, v in videos.items()}

    def _encode_geometry(self, videos: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        depth_out, normal_out = [], []
        for i in range(videos["depth"].shape[0]):
            pair = torch.cat((videos["depth"][i:i + 1], videos["normal"][i:i + 1]))
            d, n = self.codec.encode(pair).float().split(1)
            depth_out.append(d)
            normal_out.append(n)
        return {"depth": torch.cat(depth_out), "normal": torch.cat(normal_out)}

    def _geometry_noise(self, latent: torch.Tensor, name: str, *, training: bool,
                        sample_ids: Sequence[int]) -> torch.Tensor:
        sigma = self.geometry_noise_sigma
        if sigma == 0.0:
            return latent
        if training:
            noise = torch.randn(latent.shape, device=latent.device)
        else:
            draws = []
            for sample_id in sample_ids:
                generator = torch.Generator(device=latent.device)
                generator.manual_seed(_EVAL_NOISE_SEED[name] + int(sample_id))
                draws.append(torch.randn(latent.shape[1:], device=latent.device, generator=generator))
            noise = torch.stack(draws)
        return latent * (1.0 - sigma) + noise * sigma

    # ------------------------------------------------------------------- condition
    @torch.no_grad()
    def condition(self, batch: Mapping[str, Any], *, negative: bool = False,
                  drop: torch.Tensor | None = None) -> Cosmos3Condition:
        ids, mask = self._prompt(batch, negative=negative)
        if drop is not None and not negative:
            empty_ids, empty_mask = self._empty(ids.shape[0], ids.device)
            ids, mask = _select_rows(drop, empty_ids, empty_mask, ids, mask)
        return Cosmos3Condition(
            text=self._text(ids, mask), depth=batch["depth_latent"], normal=batch["normal_latent"],
            fps=torch.as_tensor(batch["fps"], dtype=torch.float32).reshape(-1))

    def _text(self, ids: torch.Tensor, mask: torch.Tensor):
        if not self.cache_text_contexts:
            return self.text_encoder(ids, mask)
        key = (ids * mask).cpu().numpy().tobytes() + mask.cpu().numpy().tobytes()
        hit = self._text_cache.get(key)
        if hit is None:
            if len(self._text_cache) > 16:
                self._text_cache.clear()
            hit = self._text_cache[key] = self.text_encoder(ids, mask)
        return hit

    def _prompt(self, batch: Mapping[str, Any], *, negative: bool):
        prefix = "negative_" if negative else ""
        ids = batch.get(f"{prefix}text_input_ids")
        if ids is None:
            if not negative:
                raise KeyError("batch has neither caption nor text_input_ids")
            return self._empty(batch["latent"].shape[0], batch["latent"].device)
        mask = batch.get(f"{prefix}text_attention_mask")
        return ids, torch.ones_like(ids, dtype=torch.bool) if mask is None else mask.bool()

    def _empty(self, batch_size: int, device: torch.device):
        ids = torch.tensor(self.empty_prompt_ids, device=device).expand(batch_size, -1)
        return ids, torch.ones_like(ids, dtype=torch.bool)

    # --------------------------------------------------------------------- outputs
    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        return self.codec.decode(latent).float()

    def visuals(self, batch: Mapping[str, Any]) -> dict[str, torch.Tensor]:
        return {name: batch[f"{name}_video"].float() for name in ("depth", "normal")
                if f"{name}_video" in batch}


def _canonical(value: torch.Tensor, *, channels: int) -> torch.Tensor:
    if value.ndim != 5 or value.shape[2] != channels:
        raise ValueError(f"expected [B, T, {channels}, H, W], got {tuple(value.shape)}")
    return value.permute(0, 2, 1, 3, 4)


def _pixels(video: torch.Tensor) -> torch.Tensor:
    video = _canonical(video, channels=3)
    return video.float() / 127.5 - 1.0 if video.dtype == torch.uint8 else video.float()


def _select_rows(select, ids_a, mask_a, ids_b, mask_b):
    """Row-wise choice between two padded id/mask pairs (``select`` picks ``a``)."""
    width = max(ids_a.shape[1], ids_b.shape[1])

    def pad(ids, mask):
        extra = width - ids.shape[1]
        return F.pad(ids, (0, extra)), F.pad(mask, (0, extra), value=False)

    (ids_a, mask_a), (ids_b, mask_b) = pad(ids_a, mask_a), pad(ids_b, mask_b)
    row = select.to(device=ids_b.device, dtype=torch.bool)[:, None]
    return torch.where(row, ids_a, ids_b), torch.where(row, mask_a, mask_b)
