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

Every entry point describes its input as a short *chunk table* (:class:`_ChunkTable`): rows of
(latent frames, per-frame sigma or none, index of the first frame, is-it-the-reference-frame),
which the table turns into token chunks, RoPE positions and — for AdaLN networks — per-token
timestep embeddings, one row at a time, so that a frame is embedded with the same row count
whether it arrives through ``forward_ar`` or through the cached rollout (their outputs must be
bit-identical).

Parity: reference ``wm/networks/cosmos3/network.py:59-568`` (module and parameter names, entry
point signatures, token order, position formula).
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass, replace

import torch
from einops import rearrange
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
    """Unpadded prompts wrapped as ``[bos?] ids eos start_of_generation`` (one 1-D tensor each)."""
    opening = [special_tokens[key] for key in ("bos_token_id",) if key in special_tokens]
    closing = [special_tokens["eos_token_id"], special_tokens["start_of_generation"]]
    packed = []
    for index in range(input_ids.shape[0]):
        ids = input_ids[index]
        if attention_mask is not None:
            ids = ids[attention_mask[index].bool()]
        packed.append(torch.cat((ids.new_tensor(opening), ids.long(), ids.new_tensor(closing))))
    return packed


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
        device = self.embed_tokens.weight.device
        prompts = pack_text_rows(input_ids, attention_mask, self.config.special_tokens)
        lengths = tuple(int(prompt.numel()) for prompt in prompts)
        # one stable width on every rank (longer prompts widen it locally), zero padded
        width = max(max(lengths), int(self.config.text_bucket_tokens or 0))
        table = torch.zeros(len(prompts), width, dtype=torch.long, device=device)
        for row, prompt in zip(table, prompts):
            row[: prompt.numel()] = prompt.to(device)
        hidden = self.embed_tokens(table)
        index = torch.arange(width, device=device, dtype=torch.float32)
        rope = self.rotary_emb(index.view(1, width, 1).expand(len(prompts), width, 3), hidden.dtype)
        per_layer = []
        for layer in self.layers:
            hidden, key, value = layer(hidden, rope)
            per_layer.append((key, value))
        return TextContext(keys=tuple(k for k, _ in per_layer), values=tuple(v for _, v in per_layer),
                           valid_lengths=torch.tensor(lengths, device=device), lengths=lengths)


@dataclass(frozen=True)
class Cosmos3Condition:
    text: TextContext
    depth: torch.Tensor
    normal: torch.Tensor
    fps: torch.Tensor

    def repeat(self, times: int) -> "Cosmos3Condition":
        """The same condition for ``times`` stacked copies of the batch."""
        if times == 1:
            return self
        tiled = {name: torch.cat([getattr(self, name)] * times) for name in ("depth", "normal", "fps")}
        return Cosmos3Condition(text=self.text.repeat(times), **tiled)

    def with_text(self, text: TextContext) -> "Cosmos3Condition":
        return replace(self, text=text)


class _PatchLayout(torch.autograd.Function):
    """The two layouts as one gather kernel each, with the cast to ``dtype`` in the same pass; the
    gradient of one is the other."""

    @staticmethod
    def forward(ctx, value, channels, height, width, patch, to_patches, dtype):
        from agentgarten_b200.ops import native

        ctx.args = (channels, height, width, patch, to_patches, value.dtype)
        native.count()
        return native.ext().patch_layout(value.contiguous(), channels, height, width, patch, to_patches,
                                         dtype == torch.bfloat16)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        from agentgarten_b200.ops import native

        channels, height, width, patch, to_patches, dtype = ctx.args
        native.count()
        back = native.ext().patch_layout(grad.contiguous(), channels, height, width, patch, not to_patches,
                                         dtype == torch.bfloat16)
        return back, None, None, None, None, None, None


def _on_kernel(value: torch.Tensor, dtype: torch.dtype) -> bool:
    import torch.autograd.forward_ad as fwAD

    from agentgarten_b200.ops import native

    both = (torch.float32, torch.bfloat16)
    return (value.is_cuda and value.dtype in both and dtype in both and native.available()
            and fwAD.unpack_dual(value).tangent is None)


def patchify(latent: torch.Tensor, patch_size: int, dtype: torch.dtype | None = None) -> torch.Tensor:
    """``[B, C, T, H, W]`` → ``[B, T, (H/p)(W/p), p*p*C]`` (patch pixels row-major, C fastest), cast
    to ``dtype`` (default: unchanged)."""
    height, width = latent.shape[-2:]
    if height % patch_size or width % patch_size:
        raise ValueError(f"latent {height}x{width} is not divisible by patch {patch_size}")
    dtype = latent.dtype if dtype is None else dtype
    if latent.dim() == 5 and _on_kernel(latent, dtype):
        return _PatchLayout.apply(latent, latent.shape[1], height, width, patch_size, True, dtype)
    return rearrange(latent.to(dtype), "b c t (h p) (w q) -> b t (h w) (p q c)", p=patch_size, q=patch_size)


def unpatchify(patches: torch.Tensor, *, channels: int, grid: tuple[int, int],
               patch_size: int, dtype: torch.dtype | None = None) -> torch.Tensor:
    dtype = patches.dtype if dtype is None else dtype
    if patches.dim() == 4 and _on_kernel(patches, dtype):
        return _PatchLayout.apply(patches, channels, grid[0] * patch_size, grid[1] * patch_size,
                                  patch_size, False, dtype)
    return rearrange(patches.to(dtype), "b t (h w) (p q c) -> b c t (h p) (w q)", h=grid[0], w=grid[1],
                     p=patch_size, q=patch_size, c=channels)


@dataclass(frozen=True)
class GeometryFrames:
    """Geometry tokens of a frame span and the RoPE positions of both token grids."""

    geometry: torch.Tensor | None
    geometry_positions: torch.Tensor | None
    rgb_positions: torch.Tensor

    def chunk(self, rgb: torch.Tensor, start: int, stop: int):
        """RGB tokens ``[B, T, N, D]`` of frames ``start:stop`` of this span, each frame followed
        by its geometry tokens → (tokens ``[B, L, D]``, positions ``[B, L, 3]``)."""
        span = slice(start, stop)
        if self.geometry is None:
            per_frame, where = rgb, self.rgb_positions[:, span]
        else:
            per_frame = torch.cat((rgb, self.geometry[:, span]), dim=2)
            where = torch.cat((self.rgb_positions[:, span], self.geometry_positions[:, span]), dim=2)
        return per_frame.flatten(1, 2), where.flatten(1, 2)


def rgb_tokens(hidden: torch.Tensor, frames: int, grid: tuple[int, int]) -> torch.Tensor:
    """The RGB tokens of every frame out of frame-major hidden states: ``[B, T, N, D]``."""
    return hidden.unflatten(1, (frames, -1))[:, :, : grid[0] * grid[1]]


class _ChunkTable:
    """Rows of an entry point's input, embedded one by one (see the module text)."""

    def __init__(self, network: "Cosmos3Network", condition: "Cosmos3Condition",
                 grid: tuple[int, int]) -> None:
        self.network, self.condition, self.grid = network, condition, grid
        self.tokens: list[torch.Tensor] = []
        self.positions: list[torch.Tensor] = []
        self.time_tokens: list[torch.Tensor | None] = []
        self.per_frame = network._tokens_per_frame(condition, grid)

    def add(self, latent: torch.Tensor, sigma: torch.Tensor | None, first: int, *,
            reference: bool = False) -> None:
        """``latent`` [B, C, T, H, W] are condition frames ``first : first + T``; ``sigma`` [B, T]
        or ``None`` for clean frames; ``reference`` marks the external first frame."""
        network, count = self.network, latent.shape[2]
        rgb = network.embed_rgb(latent, sigma, reference=reference, condition=self.condition, start=first)
        self._push(rgb, sigma, first, count, latent.shape[0])

    def add_mixed(self, latent: torch.Tensor, sigma: torch.Tensor, known: int) -> None:
        """One chunk whose first ``known`` frames are clean (the very first one being the
        reference frame) and whose other frames carry ``sigma`` [B, T]: the bidirectional input."""
        network = self.network
        clean = network.embed_rgb(latent[:, :, :known], None, condition=self.condition)
        if known and network.config.first_frame_reference_embedding:
            mark = network.first_frame_reference_embed.to(clean.dtype)
            clean = torch.cat((clean[:, :1] + mark, clean[:, 1:]), dim=1)
        noisy = network.embed_rgb(latent[:, :, known:], sigma[:, known:], condition=self.condition, start=known)
        levels = torch.cat((torch.zeros_like(sigma[:, :known]), sigma[:, known:]), dim=1)
        self._push(torch.cat((clean, noisy), dim=1), levels, 0, latent.shape[2], latent.shape[0])

    def _push(self, rgb, sigma, first, count, batch) -> None:
        frame = self.network.geometry_frames(self.condition, start=first, stop=first + count, rgb_grid=self.grid)
        tokens, positions = frame.chunk(rgb, 0, count)
        self.tokens.append(tokens)
        self.positions.append(positions)
        self.time_tokens.append(self.network._time_tokens(sigma, batch, count, self.per_frame))

    def run(self, policy, *, feature_layers: Sequence[int] = ()):
        adaln = self.network.config.timestep_conditioning == "adaln"
        return self.network.run_layers(self.tokens, self.positions, policy, feature_layers=feature_layers,
                                       time_embeddings=self.time_tokens if adaln else None)


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
        """Parameters that no released checkpoint provides start at their neutral values."""
        from agentgarten_b200.networks.lora import initialize_lora_parameters

        initialize_lora_parameters(self)
        width = self.config.hidden_size
        with torch.no_grad():
            self.geometry_modality_embed.zero_()
            self.first_frame_reference_embed.zero_()
            for layer in self.layers:
                if layer.adaln is None:
                    continue
                layer.adaln.weight.zero_()
                layer.adaln.bias.zero_()
                layer.adaln.bias[2 * width: 3 * width] = 1   # gates of the two halves open
                layer.adaln.bias[5 * width:] = 1

    # ------------------------------------------------------------------- embedding
    @property
    def dtype(self) -> torch.dtype:
        return self.proj_in.weight.dtype

    def _grid(self, latent: torch.Tensor) -> tuple[int, int]:
        patch = self.config.patch_size
        return latent.shape[-2] // patch, latent.shape[-1] // patch

    def _patches(self, latent, condition, start, stop):
        """Patch vectors of latent frames; with channel-wise geometry the depth and normal
        patches of the same frames are appended to every vector."""
        patch = self.config.patch_size
        parts = [patchify(latent, patch, self.dtype)]
        if self.config.geometry_mode == "channels":
            parts += [patchify(control[:, :, start:stop], patch, self.dtype)
                      for control in (condition.depth, condition.normal)]
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=-1)

    def embed_rgb(self, latent: torch.Tensor, sigma: torch.Tensor | None, *,
                  reference: bool = False, condition: "Cosmos3Condition | None" = None,
                  start: int = 0) -> torch.Tensor:
        """Latent frames ``[B, C, T, H, W]`` → RGB tokens ``[B, T, N, D]``.

        ``sigma`` ``[B, T]`` adds the timestep embedding; ``None`` marks clean frames.
        ``reference`` marks a chunk that is exactly the external first frame C0.
        """
        tokens = self.proj_in(self._patches(latent, condition, start, start + latent.shape[2]))
        if reference and self.config.first_frame_reference_embedding:
            tokens = tokens + self.first_frame_reference_embed.to(tokens.dtype)
        if sigma is None:
            return tokens
        return tokens + self.time_embedding(sigma)[:, :, None].to(tokens.dtype)

    def time_embedding(self, sigma: torch.Tensor) -> torch.Tensor:
        """Per-frame FP32 timestep embedding ``[B, T, D]``."""
        # two roundings, in this order, as the reference multiplies (they differ from one product
        # by the combined factor whenever timestep_scale is not a power of two)
        scaled = sigma.float().flatten() * 1000.0 * self.config.timestep_scale
        return self.time_embedder(scaled).unflatten(0, tuple(sigma.shape))

    def geometry_frames(self, condition: "Cosmos3Condition", *, start: int, stop: int,
                        rgb_grid: tuple[int, int],
                        frame_indices: torch.Tensor | None = None) -> GeometryFrames:
        """Embed geometry of condition frames ``start:stop`` and build both position grids.

        Temporal position of frame ``f`` is ``f * base_fps / fps + prompt_length + margin``;
        geometry rows/columns are rescaled onto the RGB grid.  ``frame_indices`` overrides
        the temporal indices (streaming relocates retained history).
        """
        config, device = self.config, condition.depth.device
        indices = torch.arange(start, stop, device=device) if frame_indices is None else frame_indices
        when = indices.to(device=device, dtype=torch.float32)[None]
        if config.enable_fps_modulation:
            when = when * (config.base_fps / condition.fps.float().to(device))[:, None]
        prompt_length = condition.text.valid_lengths.to(device=device, dtype=torch.float32)
        when = when + prompt_length[:, None] + config.temporal_modality_margin
        rgb_positions = _grid_positions(when, rgb_grid, rgb_grid)
        if config.geometry_mode == "channels":
            return GeometryFrames(None, None, rgb_positions)
        controls = [patchify(control[:, :, start:stop], config.patch_size, self.dtype)
                    for control in (condition.depth, condition.normal)]
        # proj_in is affine: the projection of the mean is the mean of the projections
        geometry = self.proj_in(torch.lerp(controls[0], controls[1], 0.5)) + self.geometry_modality_embed
        return GeometryFrames(geometry=geometry,
                              geometry_positions=_grid_positions(when, self._grid(condition.depth), rgb_grid),
                              rgb_positions=rgb_positions)

    def decode_velocity(self, hidden: torch.Tensor, grid: tuple[int, int]) -> torch.Tensor:
        """RGB hidden states ``[B, T, N, D]`` → latent velocity ``[B, C, T, H, W]`` (≥FP32)."""
        patches = self.proj_out(self.norm_moe_gen(hidden))
        wide = torch.promote_types(patches.dtype, torch.float32)
        return unpatchify(patches, channels=self.config.latent_channels, grid=grid,
                          patch_size=self.config.patch_size, dtype=wide)

    def _tokens_per_frame(self, condition, grid) -> int:
        per_frame = grid[0] * grid[1]
        if self.config.geometry_mode != "channels":
            rows, columns = self._grid(condition.depth)
            per_frame += rows * columns
        return per_frame

    def _time_tokens(self, sigma, batch, frames, per_frame):
        """AdaLN only: per-token timestep embedding of a chunk (clean frames use sigma 0)."""
        if self.config.timestep_conditioning != "adaln":
            return None
        if sigma is None:
            sigma = torch.zeros(batch, frames, device=self.proj_in.weight.device)
        per_frame_embedding = self.time_embedding(sigma).to(self.dtype)
        return per_frame_embedding.repeat_interleave(per_frame, dim=1)

    # --------------------------------------------------------------------- decoder
    def run_layers(self, chunks: list[torch.Tensor], positions: list[torch.Tensor],
                   attention: Attention, *, feature_layers: Sequence[int] = (),
                   time_embeddings: list | None = None):
        """Run the layer stack; returns final chunks and the chunk lists of tapped layers."""
        sharding = self.context_parallel
        lengths = [chunk.shape[1] for chunk in chunks]
        if sharding is not None:
            from .context_parallel import ContextParallelAttention

            chunks = [sharding.shard(chunk) for chunk in chunks]
            positions = [sharding.shard(position) for position in positions]
            if time_embeddings is not None:
                time_embeddings = [e if e is None else sharding.shard(e) for e in time_embeddings]
            attention = ContextParallelAttention(attention, sharding, lengths)
        ropes = [self.rotary_emb(position, chunk.dtype) for chunk, position in zip(chunks, positions, strict=True)]
        tapped = {int(index): None for index in feature_layers}
        for index, layer in enumerate(self.layers):
            chunks = layer(chunks, ropes, attention, index, time_embeddings)
            if index in tapped:
                tapped[index] = chunks
        features = [tapped[index] for index in sorted(tapped) if tapped[index] is not None]
        if sharding is not None:
            def whole(group):
                return [sharding.gather(chunk, length) for chunk, length in zip(group, lengths, strict=True)]

            chunks, features = whole(chunks), [whole(group) for group in features]
        return chunks, features

    def _text(self, text: TextContext) -> TextContext:
        return text if self.context_parallel is None else self.context_parallel.text(text)

    # --------------------------------------------------------------- bidirectional
    def forward(self, noisy: torch.Tensor, sigma: torch.Tensor, condition: Cosmos3Condition, *,
                known_frames: int = 1, feature_layers: Sequence[int] = ()):
        batch, _, frames, height, width = noisy.shape
        grid = self._grid(noisy)
        table = _ChunkTable(self, condition, grid)
        table.add_mixed(noisy, frame_sigma(sigma, batch, frames).to(noisy.device), known_frames)
        (hidden,), features = table.run(FullAttention(self._text(condition.text)), feature_layers=feature_layers)
        predicted = self.decode_velocity(rgb_tokens(hidden, frames, grid)[:, known_frames:], grid)
        still = predicted.new_zeros(batch, predicted.shape[1], known_frames, height, width)
        velocity = torch.cat((still, predicted), dim=2)
        if feature_layers:
            return velocity, tuple(group[0] for group in features)
        return velocity

    # --------------------------------------------------------- block autoregression
    def forward_ar(self, anchor: torch.Tensor, noisy: torch.Tensor, sigma: torch.Tensor,
                   condition: Cosmos3Condition, *, block_frames: int,
                   clean: torch.Tensor | None = None, history: HistoryWindow | None = None):
        batch, _, frames = noisy.shape[:3]
        if frames % block_frames:
            raise ValueError(f"{frames} target frames are not a multiple of {block_frames}")
        grid = self._grid(noisy)
        levels = frame_sigma(sigma, batch, frames).to(noisy.device)
        # rows: C0, then per block the noisy frames and (teacher forcing) their clean version
        table = _ChunkTable(self, condition, grid)
        table.add(anchor, None, 0, reference=True)
        for first in range(0, frames, block_frames):
            block = slice(first, first + block_frames)
            table.add(noisy[:, :, block], levels[:, block], first + 1)
            if clean is not None:
                table.add(clean[:, :, block], None, first + 1)
        policy = BlockCausalAttention(self._text(condition.text), teacher_forcing=clean is not None,
                                      history=history if history is not None else HistoryWindow())
        hidden, _ = table.run(policy)
        queried = hidden[1::2] if clean is not None else hidden[1:]
        return torch.cat([self.decode_velocity(rgb_tokens(chunk, block_frames, grid), grid)
                          for chunk in queried], dim=2)

    # -------------------------------------------------------------------- KV cache
    def prefill(self, anchor: torch.Tensor, condition: Cosmos3Condition, *,
                history: HistoryWindow | None = None) -> KVCache:
        grid = self._grid(anchor)
        text = self._text(condition.text)
        table = _ChunkTable(self, condition, grid)
        table.add(anchor, None, 0, reference=True)
        policy = AnchorAttention(text)
        table.run(policy)
        return KVCache(text=text, anchor=tuple(policy.recorded), condition=condition, grid=grid,
                       history=history if history is not None else HistoryWindow())

    def denoise(self, cache: KVCache, noisy: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
        hidden, _ = self._cached_chunk(cache, noisy, sigma, record=False)
        return self.decode_velocity(rgb_tokens(hidden, noisy.shape[2], cache.grid), cache.grid)

    def commit(self, cache: KVCache, clean: torch.Tensor,
               sigma: torch.Tensor | None = None) -> KVCache:
        _, recorded = self._cached_chunk(cache, clean, sigma, record=True)
        return cache.committed(tuple(recorded), clean.shape[2])

    def _cached_chunk(self, cache: KVCache, latent: torch.Tensor, sigma, *, record: bool):
        """The next block against the cache → (hidden states, recorded K/V per layer)."""
        batch, _, frames = latent.shape[:3]
        levels = None if sigma is None else frame_sigma(sigma, batch, frames).to(latent.device)
        table = _ChunkTable(self, cache.condition, cache.grid)
        table.add(latent, levels, 1 + cache.frames_committed)
        policy = CachedAttention(cache, record=record)
        (hidden,), _ = table.run(policy)
        return hidden, (policy.recorded if record else ())


def frame_sigma(sigma, batch: int, frames: int) -> torch.Tensor:
    """Broadcast a scalar, ``[B]`` or ``[B, T]`` sigma to per-frame ``[B, T]`` FP32."""
    levels = torch.as_tensor(sigma).float()
    if levels.ndim <= 1:
        levels = levels.reshape(-1, 1).expand(batch, frames)
    if tuple(levels.shape) != (batch, frames):
        raise ValueError(f"sigma must be [B] or [B, {frames}], got {tuple(levels.shape)}")
    return levels


def _grid_positions(temporal: torch.Tensor, grid: tuple[int, int],
                    rgb_grid: tuple[int, int]) -> torch.Tensor:
    """``[B, F, h*w, 3]`` positions (time, row, column); rows and columns are the pixel centres
    of ``grid`` expressed on ``rgb_grid``, so a coarser geometry grid overlays the RGB one."""
    batch, frames = temporal.shape
    rows, columns = grid

    def centres(count: int, onto: int) -> torch.Tensor:
        steps = torch.arange(count, device=temporal.device, dtype=torch.float32)
        return (steps + 0.5) * (onto / count) - 0.5

    shape = (batch, frames, rows, columns)
    axes = (temporal.view(batch, frames, 1, 1).expand(shape),
            centres(rows, rgb_grid[0]).view(1, 1, rows, 1).expand(shape),
            centres(columns, rgb_grid[1]).view(1, 1, 1, columns).expand(shape))
    return torch.stack(axes, dim=-1).reshape(batch, frames, rows * columns, 3)
