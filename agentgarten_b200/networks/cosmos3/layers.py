"""Building blocks of the Cosmos3-Nano-shaped towers.

Parameter names follow the released checkpoint (``self_attn.add_q_proj``,
``mlp_moe_gen.gate_proj`` ...), so state dicts are interchangeable.  All arithmetic goes
through :mod:`agentgarten_b200.ops`, which runs the sm_100a kernels for bf16 CUDA tensors
and the PyTorch definitions elsewhere.

A generation layer is split in two halves around attention:

``project``  RMSNorm → q/k/v projections → per-head RMSNorm(q, k) → 3-axis RoPE(q, k)
``finish``   output projection + residual → RMSNorm → SwiGLU MLP + residual

Both halves act row-wise on tokens, so a list of token chunks can be processed chunk by
chunk or as one concatenated matrix with identical per-row results.

Parity: reference ``wm/networks/cosmos3/layers.py:26-312``.
"""

from __future__ import annotations

import math
from collections.abc import Callable
from dataclasses import dataclass, field

import torch
from torch import nn

from agentgarten_b200 import ops

__all__ = [
    "Cosmos3Config",
    "Cosmos3GenLayer",
    "Cosmos3MLP",
    "Cosmos3RMSNorm",
    "Cosmos3RotaryEmbedding",
    "Cosmos3TextLayer",
    "TimestepEmbedder",
    "apply_rotary",
]


@dataclass
class Cosmos3Config:
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 151936
    rms_norm_eps: float = 1e-6
    attention_bias: bool = False
    rope_theta: float = 5_000_000.0
    mrope_section: tuple[int, int, int] = (24, 20, 20)
    latent_channels: int = 48
    patch_size: int = 2
    base_fps: float = 24.0
    enable_fps_modulation: bool = True
    temporal_modality_margin: int = 15000
    timestep_scale: float = 0.001
    # Learned type embedding added to the RGB patches of the external first frame.
    first_frame_reference_embedding: bool = True
    # Text rows are padded to this many tokens so that shapes stay stable across prompts.
    text_bucket_tokens: int | None = 514
    special_tokens: dict[str, int] = field(
        default_factory=lambda: {"eos_token_id": 151_645, "start_of_generation": 151_652})
    # "add": the timestep embedding is added to the noisy RGB tokens (released model).
    # "adaln": additionally every layer is modulated (shift/scale/gate) by the per-frame
    # timestep embedding, DiT style.
    timestep_conditioning: str = "add"
    # "tokens": depth/normal latents become extra tokens per frame (released model).
    # "channels": depth and normal latents are concatenated to the RGB latent on channels.
    geometry_mode: str = "tokens"

    def __post_init__(self) -> None:
        self.mrope_section = tuple(int(v) for v in self.mrope_section)
        if self.timestep_conditioning not in ("add", "adaln"):
            raise ValueError(f"unknown timestep_conditioning {self.timestep_conditioning!r}")
        if self.geometry_mode not in ("tokens", "channels"):
            raise ValueError(f"unknown geometry_mode {self.geometry_mode!r}")

    @property
    def patch_dim(self) -> int:
        return self.latent_channels * self.patch_size ** 2

    @property
    def input_patch_dim(self) -> int:
        return self.patch_dim * (3 if self.geometry_mode == "channels" else 1)


class Cosmos3RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(hidden_states, self.weight, self.variance_epsilon)


class Linear(nn.Linear):
    """``nn.Linear`` whose matmul runs on the tcgen05 GEMM for bf16 CUDA tensors."""

    def forward(self, value: torch.Tensor) -> torch.Tensor:
        return ops.linear(value, self.weight, self.bias)


class Cosmos3MLP(nn.Module):
    def __init__(self, config: Cosmos3Config) -> None:
        super().__init__()
        self.gate_proj = Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, value: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``down(silu(gate(value)) * up(value))``, plus ``residual`` when one is given (added in the
        down projection's epilogue where no gradient is wanted)."""
        both = ops.joint_linear(value, (self.gate_proj, self.up_proj))  # one GEMM where it applies
        act = ops.silu_mul_pair(both) if both is not None \
            else ops.silu_mul(self.gate_proj(value), self.up_proj(value))
        if residual is None:
            return self.down_proj(act)
        return ops.linear_residual(act, self.down_proj, residual)


class TimestepEmbedder(nn.Module):
    """Sinusoidal(256) features → two-layer MLP evaluated in FP32.

    The features are rounded to the parameter dtype first (what an autocast-FP32 MLP
    on bf16 features sees), then both linears run in FP32 with upcast weights.
    """

    def __init__(self, hidden_size: int, frequency_embedding_size: int = 256) -> None:
        super().__init__()
        self.linear_1 = nn.Linear(frequency_embedding_size, hidden_size, bias=True)
        self.act = nn.SiLU()
        self.linear_2 = nn.Linear(hidden_size, hidden_size, bias=True)
        self.frequency_embedding_size = frequency_embedding_size

    def forward(self, timestep: torch.Tensor) -> torch.Tensor:
        half = self.frequency_embedding_size // 2
        scale = -math.log(10_000) / half
        frequencies = torch.exp(
            scale * torch.arange(half, device=timestep.device, dtype=torch.float32))
        angle = timestep[:, None].float() * frequencies[None]
        features = torch.cat((angle.cos(), angle.sin()), dim=-1)
        features = features.to(self.linear_1.weight.dtype).float()
        with torch.autocast(timestep.device.type, enabled=False):
            hidden = self.act(ops.rows_linear(features, self.linear_1.weight, self.linear_1.bias))
            return ops.rows_linear(hidden, self.linear_2.weight, self.linear_2.bias)


class Cosmos3RotaryEmbedding(nn.Module):
    """3-axis interleaved M-RoPE tables.

    Positions are ``[B, N, 3]`` = (time, row, column).  Frequency slot ``j`` of the 64
    uses the time axis unless ``j % 3 == 1`` and ``j < 3 * section[1]`` (row axis) or
    ``j % 3 == 2`` and ``j < 3 * section[2]`` (column axis).
    """

    def __init__(self, config: Cosmos3Config) -> None:
        super().__init__()
        self.head_dim = config.head_dim
        self.rope_theta = config.rope_theta
        self.mrope_section = config.mrope_section

    def axis_of_slot(self, device: torch.device | None = None) -> torch.Tensor:
        slots = torch.arange(self.head_dim // 2, device=device)
        axis = torch.zeros_like(slots)
        for which in (1, 2):
            axis[(slots % 3 == which) & (slots < 3 * self.mrope_section[which])] = which
        return axis

    @torch.no_grad()
    def angles(self, positions: torch.Tensor) -> torch.Tensor:
        """FP32 rotation angles ``[B, N, D/2]``."""
        device = positions.device
        exponent = torch.arange(0, self.head_dim, 2, dtype=torch.float32, device=device)
        inverse = 1.0 / (self.rope_theta ** (exponent / self.head_dim))
        axis = self.axis_of_slot(device)
        picked = positions.float().index_select(-1, axis)  # [B, N, D/2]
        return picked * inverse

    @torch.no_grad()
    def forward(self, positions: torch.Tensor, dtype: torch.dtype):
        if positions.is_cuda and dtype in (torch.bfloat16, torch.float32) and self.head_dim == 128 \
                and ops.native.available():
            # one kernel: gather the axis, scale, cosine and sine (evaluated in double), cast, duplicate
            device = positions.device
            exponent = torch.arange(0, self.head_dim, 2, dtype=torch.float32, device=device)
            inverse = 1.0 / (self.rope_theta ** (exponent / self.head_dim))
            ops.native.count()
            return ops.native.ext().rope_tables(positions.float().contiguous(), inverse,
                                                self.axis_of_slot(device).int(), dtype == torch.bfloat16)
        angle = self.angles(positions)
        full = torch.cat((angle, angle), dim=-1)
        return full.cos().to(dtype), full.sin().to(dtype)


def apply_rotary(value: torch.Tensor, cosine: torch.Tensor, sine: torch.Tensor) -> torch.Tensor:
    return ops.rotary(value, cosine, sine)


class _Projections(nn.Module):
    """q/k/v/out projections and the per-head norms, under configurable attribute names."""

    def __init__(self, config: Cosmos3Config, names: tuple[str, str, str, str, str, str]) -> None:
        super().__init__()
        hidden, dim, bias = config.hidden_size, config.head_dim, config.attention_bias
        heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
        q, k, v, out, norm_q, norm_k = names
        self._names = names
        setattr(self, q, Linear(hidden, heads * dim, bias=bias))
        setattr(self, k, Linear(hidden, kv_heads * dim, bias=bias))
        setattr(self, v, Linear(hidden, kv_heads * dim, bias=bias))
        setattr(self, out, Linear(heads * dim, hidden, bias=bias))
        setattr(self, norm_q, Cosmos3RMSNorm(dim, eps=config.rms_norm_eps))
        setattr(self, norm_k, Cosmos3RMSNorm(dim, eps=config.rms_norm_eps))

    def parts(self):
        return tuple(getattr(self, name) for name in self._names)


_TEXT_NAMES = ("to_q", "to_k", "to_v", "to_out", "norm_q", "norm_k")
_GEN_NAMES = ("add_q_proj", "add_k_proj", "add_v_proj", "to_add_out", "norm_added_q", "norm_added_k")


def _project(hidden, norm, attn: _Projections, heads: int, kv_heads: int, dim: int, cos, sin):
    batch, tokens, _ = hidden.shape
    to_q, to_k, to_v, _out, norm_q, norm_k = attn.parts()
    normalized = norm(hidden)
    eps = norm_q.variance_epsilon
    # one GEMM over q | k | v where the three weights are adjacent in memory and no gradient is
    # wanted (serving after prepare_serving, frozen towers under the optimizer engine's layout)
    joint = ops.joint_linear(normalized, (to_q, to_k, to_v))
    if joint is not None:
        q_lin, k_lin, value = joint.split((heads * dim, kv_heads * dim, kv_heads * dim), dim=-1)
        query = ops.head_norm_rope(q_lin.unflatten(-1, (heads, dim)), norm_q.weight, cos, sin, eps)
        key = ops.head_norm_rope(k_lin.unflatten(-1, (kv_heads, dim)), norm_k.weight, cos, sin, eps)
        return query, key, value.unflatten(-1, (kv_heads, dim))
    query = ops.head_norm_rope(
        to_q(normalized).view(batch, tokens, heads, dim), norm_q.weight, cos, sin, eps)
    key = ops.head_norm_rope(
        to_k(normalized).view(batch, tokens, kv_heads, dim), norm_k.weight, cos, sin, eps)
    value = to_v(normalized).view(batch, tokens, kv_heads, dim)
    return query, key, value


class Cosmos3TextLayer(nn.Module):
    """Causal text-tower layer; returns its keys and values for the generation tower."""

    def __init__(self, config: Cosmos3Config) -> None:
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.self_attn = _Projections(config, _TEXT_NAMES)
        self.mlp = Cosmos3MLP(config)
        self.input_layernorm = Cosmos3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = Cosmos3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden: torch.Tensor, rope: tuple[torch.Tensor, torch.Tensor]):
        query, key, value = _project(
            hidden, self.input_layernorm, self.self_attn, self.num_attention_heads,
            self.num_key_value_heads, self.head_dim, *rope)
        output = ops.attention(query, key, value, causal=True)
        residual = hidden + self.self_attn.to_out(output.flatten(-2))
        output = residual + self.mlp(self.post_attention_layernorm(residual))
        return output, key, value


class Cosmos3GenLayer(nn.Module):
    """Generation-tower layer over a list of token chunks and one attention policy."""

    def __init__(self, config: Cosmos3Config) -> None:
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.self_attn = _Projections(config, _GEN_NAMES)
        self.mlp_moe_gen = Cosmos3MLP(config)
        self.input_layernorm_moe_gen = Cosmos3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm_moe_gen = Cosmos3RMSNorm(
            config.hidden_size, eps=config.rms_norm_eps)
        self.adaln = None
        if config.timestep_conditioning == "adaln":
            # shift/scale/gate for the attention half and for the MLP half
            self.adaln = nn.Linear(config.hidden_size, 6 * config.hidden_size, bias=True)

    # -- halves -------------------------------------------------------------------
    def project(self, hidden, cosine, sine, modulation=None):
        if modulation is not None:
            shift, scale = modulation[0], modulation[1]
            ln = self.input_layernorm_moe_gen
            norm = lambda x: ops.norm_modulate(x, ln.weight, scale, shift, ln.variance_epsilon)  # noqa: E731
        else:
            norm = self.input_layernorm_moe_gen
        return _project(hidden, norm, self.self_attn, self.num_attention_heads,
                        self.num_key_value_heads, self.head_dim, cosine, sine)

    def finish(self, hidden, attention, modulation=None):
        if modulation is None:
            residual = ops.linear_residual(attention.flatten(-2), self.self_attn.to_add_out, hidden)
            return self.mlp_moe_gen(self.post_attention_layernorm_moe_gen(residual), residual=residual)
        out = self.self_attn.to_add_out(attention.flatten(-2))
        _, _, gate_a, shift_m, scale_m, gate_m = modulation
        residual = ops.gated_residual(hidden, gate_a, out)
        ln = self.post_attention_layernorm_moe_gen
        normalized = ops.norm_modulate(residual, ln.weight, scale_m, shift_m, ln.variance_epsilon)
        return ops.gated_residual(residual, gate_m, self.mlp_moe_gen(normalized))

    def modulation(self, embedding: torch.Tensor | None):
        """``embedding`` ``[B, N, H]`` per-token timestep embedding → six ``[B, N, H]`` terms."""
        if self.adaln is None or embedding is None:
            return None
        terms = self.adaln(torch.nn.functional.silu(embedding)).to(embedding.dtype)
        return terms.chunk(6, dim=-1)

    def forward(
        self,
        chunks: list[torch.Tensor],
        ropes: list[tuple[torch.Tensor, torch.Tensor]],
        attention: Callable[..., list[torch.Tensor]],
        layer_index: int,
        time_embeddings: list[torch.Tensor | None] | None = None,
    ) -> list[torch.Tensor]:
        from agentgarten_b200.ops import fused_layer

        if time_embeddings is None and fused_layer.eligible(self, chunks, attention):
            return fused_layer.run(self, chunks, ropes, attention, layer_index)
        if time_embeddings is None and len(chunks) > 1 and ops.native.use(chunks[0]) and all(
                c.shape[0] == chunks[0].shape[0] for c in chunks):
            # Everything but attention is row-wise: run it once over the rows of all chunks
            # (one set of launches per layer instead of one per chunk) and hand attention
            # per-chunk views.  Only with the CUDA kernels, whose results do not depend on how
            # many rows are processed together (a cached rollout replays bit for bit).
            sizes = [c.shape[1] for c in chunks]
            rope = (torch.cat([r[0] for r in ropes], dim=1), torch.cat([r[1] for r in ropes], dim=1))
            hidden = torch.cat(chunks, dim=1)
            query, key, value = self.project(hidden, *rope)
            outputs = attention(layer_index, list(query.split(sizes, dim=1)),
                                list(key.split(sizes, dim=1)), list(value.split(sizes, dim=1)))
            return list(self.finish(hidden, torch.cat(outputs, dim=1)).split(sizes, dim=1))
        mods = [None] * len(chunks) if time_embeddings is None else [
            self.modulation(e) for e in time_embeddings]
        projected = [self.project(h, *rope, m) for h, rope, m in zip(chunks, ropes, mods, strict=True)]
        queries, keys, values = (list(items) for items in zip(*projected, strict=True))
        outputs = attention(layer_index, queries, keys, values)
        return [self.finish(h, o, m) for h, o, m in zip(chunks, outputs, mods, strict=True)]
