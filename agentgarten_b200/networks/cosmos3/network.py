"""Text tower and geometry-conditioned generation tower.

All entry points of :class:`Cosmos3Network` run the same layer stack over a *list of token
chunks* with one attention policy:

=================  ==============================================  ======================
entry point        chunks                                          policy
=================  ==============================================  ======================
``forward``        one chunk with every frame                      ``FullAttention``
``forward_ar``     ``[C0, noisy_1, (clean_1), noisy_2, ...]``      ``BlockCausalAttention``
``prefill``        ``[C0]``                                        ``AnchorAttention``
``denoise/commit`` one new block                                   ``CachedAttention``
=================  ==============================================  ======================

A chunk is frame-major ``[RGB_f, GEO_f]``: the RGB patches of a frame followed by the
geometry tokens of the same frame (``lerp(depth, normal, 0.5)`` through the same input
projection plus a modality embedding), each with its own 3-axis RoPE positions.  The text
prompt never becomes a token of this tower: the text tower's per-layer keys and values are
prepended to the keys of every layer.

Parity: reference ``wm/networks/cosmos3/network.py:59-568``.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass, replace

import torch
from torch import nn

from agentgarten_b200.parallel.network import ParallelNetwork
from agentgarten_b200.protocols import HistoryWindow

from .attention import (
    AnchorAttention,
    BlockCausalAttention,
    CachedAttention,
    FullAttention,
    KVCache,
    TextContext,
)
from .layers import (
    Cosmos3Config,
    Cosmos3GenLayer,
    Cosmos3RMSNorm,
    Cosmos3RotaryEmbedding,
    Cosmos3TextLayer,
    Linear,
    TimestepEmbedder,
)

__all__ = [
    "Cosmos3Condition",
    "Cosmos3Network",
    "Cosmos3TextEncoder",
    "GeometryFrames",
    "frame_sigma",
    "pack_text_rows",
    "patchify",
    "rgb_tokens",
    "unpatchify",
]

Attention = Callable[[int, list, list, list], list]


def pack_text_rows(input_ids: torch.Tensor, attention_mask: torch.Tensor | None,
                   special_tokens: dict[str, int]) -> list[torch.Tensor]:
    """Strip padding and wrap each prompt as ``[bos?] ids eos start_of_generation``."""
    if attention_mask is None:
        rows = list(input_ids.unbind(0))
    else:
        rows = [row[mask.bool()] for row, mask in zip(input_ids, attention_mask, strict=True)]
    head = [special_tokens["bos_token_id"]] if "bos_token_id" in special_tokens else []
    tail = [special_tokens["eos_token_id"], special_tokens["start_of_generation"]]
    return [torch.cat((row.new_tensor(head), row.long(), row.new_tensor(tail))) for row in rows]


class Cosmos3TextEncoder(ParallelNetwork):
    """Frozen causal text tower; its only product is the per-layer K/V of the prompt."""

    def __init__(self, config: Cosmos3Config) -> None:
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(
            Cosmos3TextLayer(config) for _ in range(config.num_hidden_layers))
        self.rotary_emb = Cosmos3RotaryEmbedding(config)

    def fsdp_units(self) -> tuple[nn.Module, ...]:
        return (self.embed_tokens,)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor,
                attention_mask: torch.Tensor | None = None) -> TextContext:
        rows = pack_text_rows(input_ids, attention_mask, self.config.special_tokens)
        lengths = tuple(int(row.numel()) for row in rows)
        bucket = max(*lengths, int(self.config.text_bucket_tokens or 0))
        device = self.embed_tokens.weight.device
        tokens = torch.zeros(len(rows), bucket, dtype=torch.long, device=device)
        for index, row in enumerate(rows):
            tokens[index, : row.numel()] = row.to(device)
        hidden = self.embed_tokens(tokens)
        steps = torch.arange(bucket, device=device, dtype=torch.float32)
        positions = steps[None, :, None].expand(len(rows), -1, 3)
        rope = self.rotary_emb(positions, hidden.dtype)
        keys, values = [], []
        for layer in self.layers:
            hidden, key, value = layer(hidden, rope)
            keys.append(key)
            values.append(value)
        return TextContext(keys=tuple(keys), values=tuple(values),
                           valid_lengths=torch.tensor(lengths, device=device), lengths=lengths)


@dataclass(frozen=True)
class Cosmos3Condition:
    text: TextContext
    depth: torch.Tensor
    normal: torch.Tensor
    fps: torch.Tensor

    def repeat(self, times: int) -> "Cosmos3Condition":
        if times == 1:
            return self
        return Cosmos3Condition(
            text=self.text.repeat(times),
            depth=torch.cat((self.depth,) * times),
            normal=torch.cat((self.normal,) * times),
            fps=torch.cat((self.fps,) * times))

    def with_text(self, text: TextContext) -> "Cosmos3Condition":
        return replace(self, text=text)


def patchify(latent: torch.Tensor, patch_size: int) -> torch.Tensor:
    """``[B, C, T, H, W]`` → ``[B, T, (H/p)(W/p), p*p*C]`` (patch pixels row-major, C fastest)."""
    b, c, t, h, w = latent.shape
    if h % patch_size or w % patch_size:
        raise ValueError(f"latent {h}x{w} is not divisible by patch {patch_size}")
    p = patch_size
    view = latent.reshape(b, c, t, h // p, p, w // p, p)
    return view.permute(0, 2, 3, 5, 4, 6, 1).reshape(b, t, (h // p) * (w // p), p * p * c)


def unpatchify(patches: torch.Tensor, *, channels: int, grid: tuple[int, int],
               patch_size: int) -> torch.Tensor:
    b, t = patches.shape[:2]
    gh, gw = grid
    p = patch_size
    view = patches.reshape(b, t, gh, gw, p, p, channels)
    return view.permute(0, 6, 1, 2, 4, 3, 5).reshape(b, channels, t, gh * p, gw * p)


@dataclass(frozen=True)
class GeometryFrames:
    """Geometry tokens of a frame span and the RoPE positions of both token grids."""

    geometry: torch.Tensor | None
    geometry_positions: torch.Tensor | None
    rgb_positions: torch.Tensor

    def chunk(self, rgb: torch.Tensor, start: int, stop: int):
        """Interleave RGB tokens ``[B, T, N, D]`` with frames ``start:stop`` → (tokens, positions)."""
        if self.geometry is None:
            return rgb.flatten(1, 2), self.rgb_positions[:, start:stop].flatten(1, 2)
        tokens = torch.cat((rgb, self.geometry[:, start:stop]), dim=2).flatten(1, 2)
        positions = torch.cat(
            (self.rgb_positions[:, start:stop], self.geometry_positions[:, start:stop]),
            dim=2).flatten(1, 2)
        return tokens, positions


def rgb_tokens(hidden: torch.Tensor, frames: int, grid: tuple[int, int]) -> torch.Tensor:
    """Pick the RGB tokens of every frame out of frame-major hidden states."""
    return hidden.unflatten(1, (frames, -1))[:, :, : grid[0] * grid[1]]


class Cosmos3Network(ParallelNetwork):
    fsdp_entry_points = ("forward_ar", "prefill", "denoise", "commit")
    context_parallel = None

    def __init__(self, config: Cosmos3Config) -> None:
        super().__init__()
        self.config = config
        self.proj_in = Linear(config.input_patch_dim, config.hidden_size, bias=True)
        self.proj_out = Linear(config.hidden_size, config.patch_dim, bias=True)
        self.time_embedder = TimestepEmbedder(config.hidden_size)
        self.norm_moe_gen = Cosmos3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.geometry_modality_embed = nn.Parameter(torch.zeros(config.hidden_size))
        self.first_frame_reference_embed = nn.Parameter(torch.zeros(config.hidden_size))
        self.layers = nn.ModuleList(
            Cosmos3GenLayer(config) for _ in range(config.num_hidden_layers))
        self.rotary_emb = Cosmos3RotaryEmbedding(config)

    # ---------------------------------------------------------------- parallel hooks
    def enable_context_parallel(self, mesh) -> None:
        from .context_parallel import ContextParallel

        self.context_parallel = ContextParallel(
            mesh, self.config.num_attention_heads, self.config.num_key_value_heads)

    def initialize_after_materialization(self) -> None:
        from agentgarten_b200.networks.lora import initialize_lora_parameters

        initialize_lora_parameters(self)
        with torch.no_grad():
            self.geometry_modality_embed.zero_()
            self.first_frame_reference_embed.zero_()
            for layer in self.layers:
                if layer.adaln is not None:
                    layer.adaln.weight.zero_()
                    layer.adaln.bias.zero_()
                    layer.adaln.bias[2 * self.config.hidden_size: 3 * self.config.hidden_size] = 1
                    layer.adaln.bias[5 * self.config.hidden_size:] = 1

    # ------------------------------------------------------------------- embedding
    @property
    def dtype(self) -> torch.dtype:
        return self.proj_in.weight.dtype

    def _patches(self, latent, condition, start, stop):
        patches = patchify(latent.to(self.dtype), self.config.patch_size)
        if self.config.geometry_mode == "channels":
            depth = patchify(condition.depth[:, :, start:stop].to(self.dtype), self.config.patch_size)
            normal = patchify(condition.normal[:, :, start:stop].to(self.dtype), self.config.patch_size)
            patches = torch.cat((patches, depth, normal), dim=-1)
        return patches

    def embed_rgb(self, latent: torch.Tensor, sigma: torch.Tensor | None, *,
                  reference: bool = False, condition: "Cosmos3Condition | None" = None,
                  start: int = 0) -> torch.Tensor:
        """Latent frames ``[B, C, T, H, W]`` → RGB tokens ``[B, T, N, D]``.

        ``sigma`` ``[B, T]`` adds the timestep embedding; ``None`` marks clean frames.
        ``reference`` marks a chunk that is exactly the external first frame C0.
        """
        frames = latent.shape[2]
        tokens = self.proj_in(self._patches(latent, condition, start, start + frames))
        if reference and self.config.first_frame_reference_embedding:
            tokens = tokens + self.first_frame_reference_embed.to(tokens.dtype)
        if sigma is not None:
            tokens = tokens + self.time_embedding(sigma)[:, :, None].to(tokens.dtype)
        return tokens

    def time_embedding(self, sigma: torch.Tensor) -> torch.Tensor:
        """Per-frame FP32 timestep embedding ``[B, T, D]``."""
        batch, frames = sigma.shape
        timestep = sigma.reshape(-1).float() * 1000.0 * self.config.timestep_scale
        return self.time_embedder(timestep).reshape(batch, frames, -1)

    def geometry_frames(self, condition: "Cosmos3Condition", *, start: int, stop: int,
                        rgb_grid: tuple[int, int],
                        frame_indices: torch.Tensor | None = None) -> GeometryFrames:
        """Embed geometry of condition frames ``start:stop`` and build both position grids.

        Temporal position of frame ``f`` is ``f * base_fps / fps + prompt_length + margin``;
        geometry rows/columns are rescaled onto the RGB grid.  ``frame_indices`` overrides
        the temporal indices (streaming relocates retained history).
        """
        config = self.config
        device = condition.depth.device
        if frame_indices is None:
            temporal = torch.arange(start, stop, device=device, dtype=torch.float32)[None]
        else:
            temporal = frame_indices.to(device=device, dtype=torch.float32)[None]
        if config.enable_fps_modulation:
            temporal = temporal * (config.base_fps / condition.fps.float().to(device))[:, None]
        origin = condition.text.valid_lengths.to(device=device, dtype=torch.float32)
        temporal = temporal + origin[:, None] + config.temporal_modality_margin
        rgb_positions = _grid_positions(temporal, rgb_grid, rgb_grid)
        if config.geometry_mode == "channels":
            return GeometryFrames(None, None, rgb_positions)
        depth = patchify(condition.depth[:, :, start:stop].to(self.dtype), config.patch_size)
        normal = patchify(condition.normal[:, :, start:stop].to(self.dtype), config.patch_size)
        # proj_in is affine: projecting the mean equals the mean of the projections.
        geometry = self.proj_in(torch.lerp(depth, normal, 0.5)) + self.geometry_modality_embed
        geometry_grid = (condition.depth.shape[-2] // config.patch_size,
                         condition.depth.shape[-1] // config.patch_size)
        return GeometryFrames(
            geometry=geometry,
            geometry_positions=_grid_positions(temporal, geometry_grid, rgb_grid),
            rgb_positions=rgb_positions)

    def decode_velocity(self, hidden: torch.Tensor, grid: tuple[int, int]) -> torch.Tensor:
        """RGB hidden states ``[B, T, N, D]`` → latent velocity ``[B, C, T, H, W]`` (≥FP32)."""
        patches = self.proj_out(self.norm_moe_gen(hidden))
        return unpatchify(
            patches.to(torch.promote_types(patches.dtype, torch.float32)),
            channels=self.config.latent_channels, grid=grid, patch_size=self.config.patch_size)

    def _tokens_per_frame(self, condition, grid) -> int:
        rgb = grid[0] * grid[1]
        if self.config.geometry_mode == "channels":
            return rgb
        p = self.config.patch_size
        return rgb + (condition.depth.shape[-2] // p) * (condition.depth.shape[-1] // p)

    def _time_tokens(self, sigma, batch, frames, per_frame):
        """AdaLN only: per-token timestep embedding of a chunk (clean frames use sigma 0)."""
        if self.config.timestep_conditioning != "adaln":
            return None
        if sigma is None:
            sigma = torch.zeros(batch, frames, device=self.proj_in.weight.device)
        embedding = self.time_embedding(sigma).to(self.dtype)
        return embedding[:, :, None].expand(-1, -1, per_frame, -1).flatten(1, 2)

    # --------------------------------------------------------------------- decoder
    def run_layers(self, chunks: list[torch.Tensor], positions: list[torch.Tensor],
                   attention: Attention, *, feature_layers: Sequence[int] = (),
                   time_embeddings: list | None = None):
        """Run the layer stack; returns final chunks and the chunk lists of tapped layers."""
        cp = self.context_parallel
        sizes = [chunk.shape[1] for chunk in chunks]
        if cp is not None:
            from .context_parallel import ContextParallelAttention

            chunks = [cp.shard(chunk) for chunk in chunks]
            positions = [cp.shard(position) for position in positions]
            if time_embeddings is not None:
                time_embeddings = [None if e is None else cp.shard(e) for e in time_embeddings]
            attention = ContextParallelAttention(attention, cp, sizes)
        ropes = [self.rotary_emb(position, chunk.dtype)
                 for chunk, position in zip(chunks, positions, strict=True)]
        wanted = frozenset(int(index) for index in feature_layers)
        features: list[list[torch.Tensor]] = []
        for index, layer in enumerate(self.layers):
            chunks = layer(chunks, ropes, attention, index, time_embeddings)
            if index in wanted:
                features.append(chunks)
        if cp is not None:
            chunks = [cp.gather(c, n) for c, n in zip(chunks, sizes, strict=True)]
            features = [[cp.gather(c, n) for c, n in zip(group, sizes, strict=True)]
                        for group in features]
        return chunks, features

    def _text(self, text: TextContext) -> TextContext:
        return text if self.context_parallel is None else self.context_parallel.text(text)

    # --------------------------------------------------------------- bidirectional
    def forward(self, noisy: torch.Tensor, sigma: torch.Tensor, condition: Cosmos3Condition, *,
                known_frames: int = 1, feature_layers: Sequence[int] = ()):
        batch, _, frames, height, width = noisy.shape
        patch = self.config.patch_size
        grid = (height // patch, width // patch)
        sigma = frame_sigma(sigma, batch, frames).to(noisy.device)
        known = self.embed_rgb(noisy[:, :, :known_frames], None, condition=condition)
        if known_frames and self.config.first_frame_reference_embedding:
            # Only the true first frame is the external reference C0.
            known = torch.cat(
                (known[:, :1] + self.first_frame_reference_embed.to(known.dtype), known[:, 1:]),
                dim=1)
        rest = self.embed_rgb(noisy[:, :, known_frames:], sigma[:, known_frames:],
                              condition=condition, start=known_frames)
        rgb = torch.cat((known, rest), dim=1)
        frame = self.geometry_frames(condition, start=0, stop=frames, rgb_grid=grid)
        tokens, positions = frame.chunk(rgb, 0, frames)
        per_frame = self._tokens_per_frame(condition, grid)
        time_tokens = None
        if self.config.timestep_conditioning == "adaln":
            mixed = torch.cat((torch.zeros_like(sigma[:, :known_frames]), sigma[:, known_frames:]), 1)
            time_tokens = [self._time_tokens(mixed, batch, frames, per_frame)]
        (hidden,), features = self.run_layers(
            [tokens], [positions], FullAttention(self._text(condition.text)),
            feature_layers=feature_layers, time_embeddings=time_tokens)
        rgb_hidden = rgb_tokens(hidden, frames, grid)
        velocity = self.decode_velocity(rgb_hidden[:, known_frames:], grid)
        velocity = torch.cat(
            (velocity.new_zeros(batch, velocity.shape[1], known_frames, height, width), velocity),
            dim=2)
        if feature_layers:
            return velocity, tuple(feature[0] for feature in features)
        return velocity

    # --------------------------------------------------------- block autoregression
    def forward_ar(self, anchor: torch.Tensor, noisy: torch.Tensor, sigma: torch.Tensor,
                   condition: Cosmos3Condition, *, block_frames: int,
                   clean: torch.Tensor | None = None, history: HistoryWindow | None = None):
        batch, _, frames, height, width = noisy.shape
        if frames % block_frames:
            raise ValueError(f"{frames} target frames are not a multiple of {block_frames}")
        patch = self.config.patch_size
        grid = (height // patch, width // patch)
        sigma = frame_sigma(sigma, batch, frames).to(noisy.device)
        per_frame = self._tokens_per_frame(condition, grid)
        chunks, positions, time_tokens = [], [], []

        def add(latent, frame_sigma_, first, reference=False):
            # Geometry is embedded per chunk, with the row count of the cached rollout.
            count = latent.shape[2]
            rgb = self.embed_rgb(latent, frame_sigma_, reference=reference,
                                 condition=condition, start=first)
            frame = self.geometry_frames(condition, start=first, stop=first + count, rgb_grid=grid)
            token, position = frame.chunk(rgb, 0, count)
            chunks.append(token)
            positions.append(position)
            time_tokens.append(self._time_tokens(frame_sigma_, batch, count, per_frame))

        add(anchor, None, 0, reference=True)
        for start in range(0, frames, block_frames):
            stop = start + block_frames
            add(noisy[:, :, start:stop], sigma[:, start:stop], start + 1)
            if clean is not None:
                add(clean[:, :, start:stop], None, start + 1)
        policy = BlockCausalAttention(self._text(condition.text),
                                      teacher_forcing=clean is not None,
                                      history=history or HistoryWindow())
        adaln = self.config.timestep_conditioning == "adaln"
        hidden, _ = self.run_layers(chunks, positions, policy,
                                    time_embeddings=time_tokens if adaln else None)
        stride = 1 if clean is None else 2
        outputs = [self.decode_velocity(rgb_tokens(chunk, block_frames, grid), grid)
                   for chunk in hidden[1::stride]]
        return torch.cat(outputs, dim=2)

    # -------------------------------------------------------------------- KV cache
    def prefill(self, anchor: torch.Tensor, condition: Cosmos3Condition, *,
                history: HistoryWindow | None = None) -> KVCache:
        patch = self.config.patch_size
        grid = (anchor.shape[-2] // patch, anchor.shape[-1] // patch)
        frame = self.geometry_frames(condition, start=0, stop=1, rgb_grid=grid)
        token, position = frame.chunk(
            self.embed_rgb(anchor, None, reference=True, condition=condition), 0, 1)
        text = self._text(condition.text)
        policy = AnchorAttention(text)
        per_frame = self._tokens_per_frame(condition, grid)
        time_tokens = self._time_tokens(None, anchor.shape[0], 1, per_frame)
        self.run_layers([token], [position], policy,
                        time_embeddings=None if time_tokens is None else [time_tokens])
        return KVCache(text=text, anchor=tuple(policy.recorded),
                       history=history or HistoryWindow(), condition=condition, grid=grid)

    def denoise(self, cache: KVCache, noisy: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
        hidden = self._cached_chunk(cache, noisy, sigma, record=None)
        return self.decode_velocity(rgb_tokens(hidden, noisy.shape[2], cache.grid), cache.grid)

    def commit(self, cache: KVCache, clean: torch.Tensor,
               sigma: torch.Tensor | None = None) -> KVCache:
        recorded: list[tuple[torch.Tensor, torch.Tensor]] = []
        self._cached_chunk(cache, clean, sigma, record=recorded)
        return cache.committed(tuple(recorded), clean.shape[2])

    def _cached_chunk(self, cache: KVCache, latent: torch.Tensor, sigma, *, record):
        batch, _, frames = latent.shape[:3]
        start = 1 + cache.frames_committed
        condition = cache.condition
        frame = self.geometry_frames(condition, start=start, stop=start + frames,
                                     rgb_grid=cache.grid)
        per_frame_sigma = None if sigma is None else \
            frame_sigma(sigma, batch, frames).to(latent.device)
        rgb = self.embed_rgb(latent, per_frame_sigma, condition=condition, start=start)
        token, position = frame.chunk(rgb, 0, frames)
        policy = CachedAttention(cache, record=record is not None)
        time_tokens = self._time_tokens(per_frame_sigma, batch, frames,
                                        self._tokens_per_frame(condition, cache.grid))
        (hidden,), _ = self.run_layers(
            [token], [position], policy,
            time_embeddings=None if time_tokens is None else [time_tokens])
        if record is not None:
            record.extend(policy.recorded)
        return hidden


def frame_sigma(sigma, batch: int, frames: int) -> torch.Tensor:
    """Broadcast a scalar, ``[B]`` or ``[B, T]`` sigma to per-frame ``[B, T]`` FP32."""
    sigma = torch.as_tensor(sigma).float()
    if sigma.ndim == 0:
        sigma = sigma.expand(batch)
    if sigma.ndim == 1:
        sigma = sigma[:, None].expand(batch, frames)
    if tuple(sigma.shape) != (batch, frames):
        raise ValueError(f"sigma must be [B] or [B, {frames}], got {tuple(sigma.shape)}")
    return sigma


def _grid_positions(temporal: torch.Tensor, grid: tuple[int, int],
                    rgb_grid: tuple[int, int]) -> torch.Tensor:
    """``[B, F, h*w, 3]`` positions; rows/cols are pixel centres rescaled to the RGB grid."""
    batch, frames = temporal.shape
    h, w = grid
    device = temporal.device
    rows = (torch.arange(h, device=device, dtype=torch.float32) + 0.5) * (rgb_grid[0] / h) - 0.5
    cols = (torch.arange(w, device=device, dtype=torch.float32) + 0.5) * (rgb_grid[1] / w) - 0.5
    out = torch.empty(batch, frames, h, w, 3, device=device, dtype=torch.float32)
    out[..., 0] = temporal[:, :, None, None]
    out[..., 1] = rows[None, None, :, None]
    out[..., 2] = cols[None, None, None, :]
    return out.reshape(batch, frames, h * w, 3)
