"""Discriminator head on frozen backbone features.

For every tapped backbone layer a branch pools the token sequence into one vector with a
learned-query cross-attention (written with explicit einsum + softmax: one query per sample
is cheap, and unlike fused attention kernels it supports the double backward that exact
R1/R2 needs) followed by a GELU MLP; the branch outputs are concatenated, layer-normed and
projected to one logit per sample.  Initialisation is seeded and independent of the memory
layout, so every rank builds the same head.

Parity: reference ``wm/networks/discriminator.py:21-193``.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist
from torch import Tensor, nn

from agentgarten_b200.parallel.engine import ParallelConfig

__all__ = ["DiscriminatorHead"]


class _RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.eps = float(eps)
        self.weight = nn.Parameter(torch.ones(int(dim)))

    def forward(self, value: Tensor) -> Tensor:
        # statistics in at least FP32 (and never a downcast of FP64 inputs)
        working = value.to(torch.promote_types(value.dtype, torch.float32))
        scale = torch.rsqrt(working.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return (working * scale).to(value) * self.weight


class _QueryPool(nn.Module):
    """A learned query attends over the tokens of one tapped layer and returns one vector per
    sample.  The attention is spelled out with matrix products and a softmax: one query per
    sample is cheap, and unlike fused attention kernels this supports the double backward that
    exact R1/R2 takes through the head."""

    def __init__(self, hidden: int, heads: int) -> None:
        super().__init__()
        if hidden % heads:
            raise ValueError("discriminator hidden size must be divisible by heads")
        self.num_heads, self.head_dim = heads, hidden // heads
        self.query_token = nn.Parameter(torch.empty(1, 1, 1, hidden))
        self.to_q = nn.Linear(hidden, hidden, bias=False)
        self.to_k = nn.Linear(hidden, hidden, bias=False)
        self.to_v = nn.Linear(hidden, hidden, bias=False)
        self.pre_norm_kv = _RMSNorm(hidden)
        self.post_norm_q = _RMSNorm(hidden)
        self.post_norm_k = _RMSNorm(hidden)
        self.to_out = nn.Linear(hidden, hidden)

    def _per_head(self, rows: Tensor) -> Tensor:
        """[B, N, hidden] → [B, heads, N, head_dim]"""
        return rows.unflatten(-1, (self.num_heads, self.head_dim)).transpose(1, 2)

    def forward(self, features: Tensor) -> Tensor:
        # in the head's own precision: the paired and penalty terms live on small differences
        tokens = self.pre_norm_kv(features.to(self.to_k.weight.dtype))
        seed = self.query_token[:, 0].expand(tokens.shape[0], -1, -1)            # [B, 1, hidden]
        query = self._per_head(self.post_norm_q(self.to_q(seed)))
        key = self._per_head(self.post_norm_k(self.to_k(tokens)))
        value = self._per_head(self.to_v(tokens))
        weights = torch.softmax(query @ key.transpose(-1, -2) * self.head_dim ** -0.5, dim=-1)
        pooled = (weights @ value).transpose(1, 2).flatten(-2)                   # [B, 1, hidden]
        return (self.to_out(pooled) + seed).squeeze(1)


class _MLP(nn.Module):
    def __init__(self, hidden: int, ratio: float) -> None:
        super().__init__()
        inner = int(hidden * ratio)
        self.norm = _RMSNorm(hidden)
        self.fc1 = nn.Linear(hidden, inner)
        self.activation = nn.GELU()
        self.fc2 = nn.Linear(inner, hidden)

    def forward(self, value: Tensor) -> Tensor:
        update = self.fc2(self.activation(self.fc1(self.norm(value))))
        return value + update


class _Branch(nn.Module):
    def __init__(self, hidden: int, ratio: float, heads: int) -> None:
        super().__init__()
        self.cross_attention = _QueryPool(hidden, heads)
        self.mlp = _MLP(hidden, ratio)

    def forward(self, features: Tensor) -> Tensor:
        return self.mlp(self.cross_attention(features))


class DiscriminatorHead(nn.Module):
    def __init__(self, *, hidden_size: int = 4096, feature_layers: Sequence[int] = (11, 23, 35),
                 mlp_ratio: float = 4.0, num_heads: int = 32, initial_logit_sign: float = 1.0,
                 seed: int = 0xD2D20000, init_device: str = "cpu") -> None:
        super().__init__()
        taps = sorted(int(index) for index in feature_layers)
        if not taps or len(taps) != len(set(taps)):
            raise ValueError(f"feature_layers must be unique and non-empty: {feature_layers}")
        if initial_logit_sign not in (-1.0, 1.0):
            raise ValueError("initial_logit_sign must be -1 or 1")
        self.feature_layers = tuple(taps)
        self.initial_logit_sign = float(initial_logit_sign)
        self.seed = int(seed)
        joined = hidden_size * len(taps)
        with torch.device(init_device):
            self.branches = nn.ModuleList(_Branch(hidden_size, mlp_ratio, num_heads) for _ in taps)
            self.final_norm = nn.LayerNorm(joined, eps=1e-6)
            self.final_linear = nn.Linear(joined, 1)
        if all(not parameter.is_meta for parameter in self.parameters()):
            self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, shard_index: int = 0) -> None:
        """Seeded and independent of the memory layout, so that every rank builds the same head:
        modules are visited in registration order and draw from one generator — Xavier-uniform
        matrices (zero biases), N(0, 0.02) query tokens; norms start at one."""
        draws = torch.Generator(device=self.final_linear.weight.device)
        draws.manual_seed(self.seed + int(shard_index))

        def xavier_(linear: nn.Linear) -> None:
            rows, columns = linear.weight.shape
            limit = (6.0 / float(rows + columns)) ** 0.5
            linear.weight.uniform_(-limit, limit, generator=draws)
            if linear.bias is not None:
                linear.bias.zero_()

        def unit_(norm: nn.Module) -> None:
            norm.weight.fill_(1.0)
            if getattr(norm, "bias", None) is not None:
                norm.bias.zero_()

        for module in self.modules():
            if isinstance(module, nn.Linear):
                xavier_(module)
            elif isinstance(module, (_RMSNorm, nn.LayerNorm)):
                unit_(module)
            elif isinstance(module, _QueryPool):
                module.query_token.normal_(0.0, 0.02, generator=draws)
        self.final_linear.weight.mul_(self.initial_logit_sign)

    def parallelize(self, config: ParallelConfig, device) -> None:
        """Place the head (small: replicated on every rank; its optimizer state is sharded by
        the optimizer engine).  Without a process-wide seed the parameters are broadcast."""
        device = torch.device(device)
        dtype = getattr(torch, config.parameter_dtype)
        on_meta = any(p.is_meta for p in self.parameters())
        if on_meta:
            self.to(dtype=dtype)
            self.to_empty(device=device)
            self.reset_parameters(0)
        else:
            self.to(device=device, dtype=dtype)
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                for p in self.parameters():
                    dist.broadcast(p.detach(), src=0)

    def _logits(self, features: Sequence[Tensor]) -> Tensor:
        if len(features) != len(self.branches):
            raise ValueError("feature count does not match discriminator branches")
        joined = torch.cat([b(f) for b, f in zip(self.branches, features, strict=True)], -1)
        return self.final_linear(self.final_norm(joined))

    def forward(self, feature_groups: Sequence[Sequence[Tensor]]) -> Tensor:
        return torch.cat([self._logits(g) for g in feature_groups]).float().reshape(-1)
