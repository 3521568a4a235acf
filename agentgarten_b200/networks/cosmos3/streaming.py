"""Block-by-block streaming sampler with a bounded KV cache.

``Cosmos3Stream`` owns one sample: ``start`` prefills the clean anchor frame, ``denoise``
predicts the velocity of the next block against the committed history without changing it,
``commit`` publishes a clean block.  The history is bounded: the first ``sink_frames``
frames stay forever, behind them a FIFO of ``history_frames``; when a commit overflows the
budget the oldest frames are evicted and the retained keys are re-rotated to their new
temporal positions (``StreamRoPE``), which keeps positions inside the range seen in
training for arbitrarily long streams.

On a B200 every layer of a step runs on the CUDA kernels over fixed K/V arenas; when the
network was prepared with ``prepare_serving(..., cuda_graphs=True)`` the whole step (all
layers, cache writes, attention and the output projection) is captured once per cache fill
level and replayed as a single CUDA graph — in steady state one graph per call.

Parity: reference ``wm/networks/cosmos3/streaming.py:20-368``.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import StrEnum

import torch

from .attention import TextContext
from .layers import apply_rotary
from .network import Cosmos3Condition, Cosmos3Network, frame_sigma, rgb_tokens, unpatchify
from .streaming_attention import StreamAttentionCache

__all__ = ["Cosmos3Stream", "StreamPolicy", "StreamRoPE"]


class StreamRoPE(StrEnum):
    """How retained history and the next query are placed on the time axis."""

    ABSOLUTE = "absolute"        # true frame indices (unbounded streams only make sense here)
    CONTIGUOUS = "contiguous"    # history slides down so that it stays contiguous after the sink
    TOP_ALIGNED = "top_aligned"  # the current block always sits at the end of the training range


@dataclass(frozen=True, slots=True)
class StreamPolicy:
    """Frame budgets exclude the current block; ``sink_frames`` counts C0 first."""

    block_frames: int = 4
    sink_frames: int = 5
    history_frames: int | None = 44
    rope: StreamRoPE = StreamRoPE.TOP_ALIGNED
    train_frames: int = 61

    def __post_init__(self) -> None:
        object.__setattr__(self, "rope", StreamRoPE(self.rope))
        if self.block_frames < 1 or self.sink_frames < 0:
            raise ValueError("block_frames must be positive and sink_frames nonnegative")
        if self.sink_frames and (self.sink_frames - 1) % self.block_frames:
            raise ValueError("sink_frames must be C0 plus complete generated blocks")
        if self.history_frames is None:
            if self.rope is not StreamRoPE.ABSOLUTE:
                raise ValueError("unbounded history requires absolute RoPE")
        elif self.history_frames < 0 or self.capacity < 1:
            raise ValueError("history_frames must be nonnegative and capacity positive")
        if self.rope is StreamRoPE.TOP_ALIGNED:
            if self.train_frames < self.capacity + self.block_frames:
                raise ValueError("train_frames must contain history and the current block")
            if (self.train_frames - 1) % self.block_frames:
                raise ValueError("train_frames must follow the C0 + N * block_frames layout")

    @property
    def capacity(self) -> int:
        if self.history_frames is None:
            raise ValueError("unbounded streams have no fixed capacity")
        return self.sink_frames + self.history_frames

    def positions(self, frames: tuple[int, ...], next_frame: int) -> tuple[int, ...]:
        """Temporal positions of absolute frame ids when the next block starts at
        ``next_frame``; sink frames never move."""
        if self.rope is StreamRoPE.ABSOLUTE:
            return frames
        if self.rope is StreamRoPE.CONTIGUOUS:
            shift = max(0, next_frame - self.capacity)
        else:
            shift = max(0, next_frame + self.block_frames - self.train_frames)
        return tuple(f if f < self.sink_frames else f - shift for f in frames)


class _StepGraph:
    """One captured denoise/commit step for a fixed cache fill level."""

    def __init__(self, stream: "Cosmos3Stream", tokens, positions_rope, record: bool, frames: int):
        self.tokens = tokens.clone()
        self.cos, self.sin = positions_rope[0].clone(), positions_rope[1].clone()
        self.graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up: fills schedule / tensor-map caches outside capture
                stream._layers_and_decode(self.tokens, (self.cos, self.sin), record, frames,
                                          advance=False)
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(self.graph, pool=stream._graph_pool):
            self.output = stream._layers_and_decode(self.tokens, (self.cos, self.sin), record,
                                                    frames, advance=False)

    def __call__(self, tokens, rope):
        self.tokens.copy_(tokens)
        self.cos.copy_(rope[0])
        self.sin.copy_(rope[1])
        self.graph.replay()
        return self.output


class Cosmos3Stream:
    """One sequential latent stream; ``reset`` reuses the model and captured graphs' pool."""

    def __init__(self, network: Cosmos3Network, policy: StreamPolicy, *,
                 initial_capacity_frames: int = 256, cuda_graphs: bool | None = None) -> None:
        if initial_capacity_frames < 1:
            raise ValueError("initial_capacity_frames must be positive")
        self.network = network
        self.policy = policy
        self.initial_capacity_frames = initial_capacity_frames
        serving = getattr(network, "_serving_options", None) or {}
        self.cuda_graphs = bool(serving.get("cuda_graphs", False)) if cuda_graphs is None \
            else bool(cuda_graphs)
        self._graph_pool = None
        self._status_probe = None  # (pinned host copy of the kernel status word, its copy event)
        self.reset()

    def reset(self, release: bool = False) -> None:
        """Forget the semantic history.  A bounded stream keeps its K/V arenas and the step
        graphs captured over them, so the next ``start`` with a prompt of the same length and
        the same frame geometry replays them at once; ``release=True`` (and any change of
        prompt length or geometry) frees both."""
        keep = (not release and getattr(self, "layers", None)
                and self.policy.history_frames is not None)
        self.text: TextContext | None = None
        if keep:
            for layer in self.layers:
                layer.clear()
        else:
            self.layers: list[StreamAttentionCache] = []
            self._graphs: dict[tuple, _StepGraph] = {}
        self.frame_ids: tuple[int, ...] = ()
        self.next_frame = 0
        self.positions: torch.Tensor | None = None
        self.grid = (0, 0)

    @torch.inference_mode()
    def capture_graphs(self, anchor: torch.Tensor, anchor_condition: Cosmos3Condition,
                       block_condition: Cosmos3Condition) -> None:
        """Runs the stream once over enough blocks to visit every cache fill level (and both
        arenas of the full cache), so that all step graphs exist before the first real block;
        ends with a ``reset`` that keeps them.  Needs a bounded policy and CUDA graphs."""
        policy = self.policy
        if not self.cuda_graphs or policy.history_frames is None:
            return
        self.reset()
        self.start(anchor, anchor_condition)
        shape = list(anchor.shape)
        shape[2] = policy.block_frames
        block = torch.zeros(shape, device=anchor.device, dtype=anchor.dtype)
        sigma = torch.ones((1,), device=anchor.device)
        fills = -(-max(policy.capacity - 1, 0) // policy.block_frames)  # blocks until the cache is full
        for _ in range(fills + 3):
            self.denoise(block, sigma, block_condition)
            self.commit(block, block_condition)
        self.reset()

    @property
    def keys(self) -> list[torch.Tensor]:
        return [layer.visual_key for layer in self.layers]

    @property
    def values(self) -> list[torch.Tensor]:
        return [layer.visual_value for layer in self.layers]

    # ----------------------------------------------------------------------- public
    @torch.inference_mode()
    def start(self, anchor: torch.Tensor, condition: Cosmos3Condition) -> None:
        """Prefill the clean first frame C0 with its matching condition."""
        if self.next_frame:
            raise RuntimeError("reset the stream before starting a new anchor")
        if anchor.shape[2] != 1:
            raise ValueError("anchor must contain exactly one latent frame")
        if anchor.shape[0] != 1:
            raise ValueError("a serving stream owns exactly one sample")
        if condition.depth.shape[2] != 1 or condition.normal.shape != condition.depth.shape:
            raise ValueError("anchor condition must contain exactly one latent frame")
        if condition.text.batch_size != 1:
            raise ValueError("a serving stream needs one text context")
        self.text = condition.text
        patch = self.network.config.patch_size
        self.grid = (anchor.shape[-2] // patch, anchor.shape[-1] // patch)
        signature = (self.grid, self.text.lengths[0], tuple(condition.depth.shape[-2:]), anchor.dtype)
        if self.layers:  # arenas kept by reset(): reusable only for the same geometry and prompt length
            if signature == self._arena_signature and len(self.layers) == len(self.text.keys):
                n, heads = self.text.lengths[0], self._local_kv_heads()
                for layer, key, value in zip(self.layers, self.text.keys, self.text.values):
                    layer.update_text(key[:, :n, heads], value[:, :n, heads])
            else:
                self.reset(release=True)
                self.text = condition.text
                self.grid = signature[0]
        self._arena_signature = signature
        self._run(anchor, None, condition, record=True, reference=True)
        self.next_frame = 1
        self.frame_ids = (0,)

    @torch.inference_mode()
    def denoise(self, noisy: torch.Tensor, sigma: torch.Tensor,
                condition: Cosmos3Condition) -> torch.Tensor:
        """Velocity of the next block; the committed history is left untouched."""
        self.validate_chunk(noisy, condition)
        return self._run(noisy, sigma, condition, record=False)

    @torch.inference_mode()
    def commit(self, clean: torch.Tensor, condition: Cosmos3Condition) -> None:
        """Publish one clean block, then evict and relocate history for the next one."""
        self.validate_chunk(clean, condition)
        self._run(clean, None, condition, record=True)
        count = clean.shape[2]
        self.frame_ids += tuple(range(self.next_frame, self.next_frame + count))
        self.next_frame += count
        self._trim(condition)
        self._check_kernel_status(clean.device)

    def _check_kernel_status(self, device: torch.device) -> None:
        """Block boundary: raise if a bounded wait ran out in any kernel of an earlier block.
        The status word is copied to pinned host memory without stalling the stream; the copy
        queued at the previous boundary is the one that is read, so a failure surfaces one
        block late at the latest and a healthy stream never synchronises here."""
        if device.type != "cuda":
            return
        from agentgarten_b200.ops import kernel_status

        if self._status_probe is not None:
            host, event = self._status_probe
            if event.query():
                kernel_status.raise_for_status(int(host.item()), "Cosmos3Stream block")
        host = torch.empty((), dtype=torch.float32).pin_memory() if self._status_probe is None \
            else self._status_probe[0]
        host.copy_(kernel_status.status_flag(device), non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._status_probe = (host, event)

    def validate_chunk(self, value: torch.Tensor, condition: Cosmos3Condition) -> None:
        if self.text is None:
            raise RuntimeError("start the stream before denoising or committing")
        if value.shape[2] != self.policy.block_frames:
            raise ValueError("current latent must contain one complete block")
        if condition.depth.shape[2] != value.shape[2] or condition.normal.shape != condition.depth.shape:
            raise ValueError("condition must contain exactly the current block")
        if condition.text is not self.text:
            raise ValueError("update_text explicitly before changing stream text")

    @torch.inference_mode()
    def update_text(self, text: TextContext) -> None:
        """Swap in another prepared prompt of the same length; visual history stays."""
        if self.text is None:
            raise RuntimeError("start the stream before updating text")
        if text.lengths != self.text.lengths or len(text.keys) != len(self.text.keys):
            raise ValueError("prompt changes must preserve text lengths and layer count")
        pairs = list(zip((*self.text.keys, *self.text.values), (*text.keys, *text.values), strict=True))
        if any(a.shape != b.shape or a.dtype != b.dtype or a.device != b.device for a, b in pairs):
            raise ValueError("prompt changes must preserve the complete text cache layout")
        for mine, theirs in pairs:
            mine.copy_(theirs)
        n = text.lengths[0]
        heads = self._local_kv_heads()
        for layer, key, value in zip(self.layers, text.keys, text.values, strict=True):
            layer.update_text(key[:, :n, heads], value[:, :n, heads])

    # -------------------------------------------------------------------- internals
    def embed_chunk(self, latent: torch.Tensor, sigma: torch.Tensor | None,
                    condition: Cosmos3Condition, *, reference: bool = False):
        """Embed the next chunk at its stream positions → ``(tokens, positions)``."""
        count = latent.shape[2]
        where = self.policy.positions(tuple(range(self.next_frame, self.next_frame + count)),
                                      self.next_frame)
        frame = self.network.geometry_frames(
            condition, start=0, stop=count, rgb_grid=self.grid,
            frame_indices=torch.arange(where[0], where[0] + count, device=latent.device))
        per_frame = None if sigma is None else \
            frame_sigma(sigma, latent.shape[0], count).to(latent.device)
        rgb = self.network.embed_rgb(latent, per_frame, reference=reference, condition=condition)
        return frame.chunk(rgb, 0, count)

    def _cache(self, index: int, key: torch.Tensor, frames_in_chunk: int) -> StreamAttentionCache:
        n = self.text.lengths[0]
        bounded = self.policy.history_frames is not None
        if index == len(self.layers):
            heads = self._local_kv_heads()
            self.layers.append(StreamAttentionCache(
                self.text.keys[index][:, :n, heads], self.text.values[index][:, :n, heads],
                key.shape[1] // frames_in_chunk,
                self.policy.capacity if bounded else self.initial_capacity_frames,
                self.policy.block_frames))
        layer = self.layers[index]
        if layer.frames + frames_in_chunk > layer.capacity + layer.block_frames:
            bigger = StreamAttentionCache(
                layer.key[:, :n], layer.value[:, :n], layer.frame_tokens,
                max(layer.capacity * 2, layer.frames + frames_in_chunk), layer.block_frames)
            bigger.append(layer.visual_key, layer.visual_value)
            layer = self.layers[index] = bigger
        return layer

    def _local_kv_heads(self) -> slice:
        """KV heads cached on this rank: all of them, or this rank's share under tensor parallelism."""
        plan = getattr(self.network, "_tensor_parallel", None)
        return slice(None) if plan is None else plan.kv_slice

    def _layers_and_decode(self, tokens, rope, record: bool, frames: int, *, advance: bool = True):
        """All layers over one chunk + output projection.  ``advance=False`` leaves the frame
        counters alone (used while capturing, the caller advances them once per real call)."""
        network = self.network

        def attend(index, queries, keys, values):
            layer = self._cache(index, keys[0], frames)
            out = layer.attend(queries[0], keys[0], values[0])
            if record and advance:
                layer.frames += frames  # the tail written by attend() becomes history
            return [out]

        plan = getattr(network, "_tensor_parallel", None)
        if plan is not None:
            # Heads and MLP columns are split over the ranks; every rank gets all output rows.
            patches = plan.run(tokens, rope, attend)
            if record:
                return patches
            config = network.config
            rgb = rgb_tokens(patches, frames, self.grid)
            return unpatchify(rgb.float(), channels=config.latent_channels, grid=self.grid,
                              patch_size=config.patch_size)
        hidden = tokens
        for index, block in enumerate(network.layers):
            (hidden,) = block([hidden], [rope], attend, index)
        if record:
            return hidden
        return network.decode_velocity(rgb_tokens(hidden, frames, self.grid), self.grid)

    def _run(self, latent, sigma, condition, *, record: bool, reference: bool = False):
        tokens, positions = self.embed_chunk(latent, sigma, condition, reference=reference)
        rope = self.network.rotary_emb(positions, tokens.dtype)
        frames = latent.shape[2]
        filled = self.layers[0].frames if self.layers else 0
        use_graph = (self.cuda_graphs and tokens.is_cuda and not reference
                     and len(self.layers) == len(self.network.layers)
                     and self.policy.history_frames is not None
                     and self.network.config.timestep_conditioning == "add")
        if use_graph:
            # arenas swap on every eviction, so the arena address is part of the key
            key = (filled, record, frames, tuple(tokens.shape), self.layers[0].key.data_ptr())
            graph = self._graphs.get(key)
            if graph is None:
                if self._graph_pool is None:
                    self._graph_pool = torch.cuda.graph_pool_handle()
                graph = self._graphs[key] = _StepGraph(self, tokens, rope, record, frames)
            out = graph(tokens, rope)
            if record:
                for layer in self.layers:
                    layer.frames += frames
            out = None if record else out.clone()
        else:
            if self.network.config.timestep_conditioning == "adaln":
                out = self._run_adaln(tokens, positions, sigma, latent, record)
            else:
                out = self._layers_and_decode(tokens, rope, record, frames)
        if record:
            self.positions = positions if self.positions is None \
                else torch.cat((self.positions, positions), 1)
            return None
        return out

    def _run_adaln(self, tokens, positions, sigma, latent, record):
        network, frames = self.network, latent.shape[2]
        per_frame = None if sigma is None else frame_sigma(sigma, 1, frames).to(latent.device)
        time_tokens = network._time_tokens(per_frame, 1, frames, tokens.shape[1] // frames)

        def attend(index, queries, keys, values):
            layer = self._cache(index, keys[0], frames)
            out = layer.attend(queries[0], keys[0], values[0])
            if record:
                layer.frames += frames
            return [out]

        (hidden,), _ = network.run_layers([tokens], [positions], attend, time_embeddings=[time_tokens])
        if record:
            return hidden
        return network.decode_velocity(rgb_tokens(hidden, frames, self.grid), self.grid)

    def _trim(self, condition: Cosmos3Condition) -> None:
        """Evict frames beyond the budget; re-rotate retained keys to their new positions."""
        policy = self.policy
        if policy.history_frames is None:
            return
        count, capacity, sink = len(self.frame_ids), policy.capacity, policy.sink_frames
        if count <= capacity:
            return
        evicted = count - capacity
        frame_tokens = self.layers[0].frame_tokens
        device = self.layers[0].key.device
        keep = torch.cat((torch.arange(sink, device=device),
                          torch.arange(sink + evicted, count, device=device)))
        self.frame_ids = self.frame_ids[:sink] + self.frame_ids[sink + evicted:]

        def retain(rows: torch.Tensor) -> torch.Tensor:
            return rows.unflatten(1, (count, frame_tokens)).index_select(1, keep).flatten(1, 2)

        old = retain(self.positions)
        if policy.rope is StreamRoPE.ABSOLUTE:
            for layer in self.layers:
                layer.replace_visual(retain(layer.visual_key), retain(layer.visual_value))
            self.positions = old
            return
        # New temporal coordinate of every retained frame for the *next* block.
        target = policy.positions(self.frame_ids, self.next_frame)
        times = torch.arange(sink, device=device).float()
        if sink < capacity:
            moved = torch.arange(target[sink], target[sink] + capacity - sink, device=device).float()
            times = torch.cat((times, moved))
        config = self.network.config
        if config.enable_fps_modulation:
            times = times * (config.base_fps / condition.fps.float().to(device))
        new = old.clone().unflatten(1, (capacity, frame_tokens))
        new[..., 0] = (times + self.text.lengths[0] + config.temporal_modality_margin)[None, :, None]
        new = new.flatten(1, 2)
        dtype = self.layers[0].key.dtype
        old_c, old_s = (t.float() for t in self.network.rotary_emb(old, dtype))
        new_c, new_s = (t.float() for t in self.network.rotary_emb(new, dtype))
        # Rotation by (new - old), built from the *rounded* tables the keys were rotated
        # with; cos(new - old) computed directly loses accuracy at large position offsets.
        norm = old_c.square() + old_s.square()
        cosine = (new_c * old_c + new_s * old_s) / norm
        sine = (new_s * old_c - new_c * old_s) / norm
        fused = self.layers[0].key.is_cuda and dtype == torch.bfloat16 \
            and self.layers[0].key.shape[-1] == 128
        for layer in self.layers:
            if fused:
                layer.relocate(sink, evicted, (cosine, sine))
                continue
            key = retain(layer.visual_key)
            rotated = apply_rotary(key.float(), cosine, sine).to(dtype)
            rotated[:, : sink * frame_tokens] = key[:, : sink * frame_tokens]
            layer.replace_visual(rotated, retain(layer.visual_value))
        self.positions = new
