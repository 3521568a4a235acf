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
        wide = value.to(torch.promote_types(value.dtype, torch.float32))
        wide = wide * torch.rsqrt(wide.square().mean(-1, keepdim=True) + self.eps)
        return wide.to(value) * self.weight


class _QueryPool(nn.Module):
    """One learned query attends over the feature tokens of a layer."""

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

    def forward(self, features: Tensor) -> Tensor:
        # work in the head's dtype: the paired and penalty terms live on small differences
        features = features.to(self.to_k.weight.dtype)
        b, n = features.shape[:2]
        start = self.query_token[:, 0].expand(b, -1, -1)
        q = self.post_norm_q(self.to_q(start)).view(b, 1, self.num_heads, -1)
        normed = self.pre_norm_kv(features)
        k = self.post_norm_k(self.to_k(normed)).view(b, n, self.num_heads, -1)
        v = self.to_v(normed).view(b, n, self.num_heads, -1)
        weights = (torch.einsum("bqhd,bkhd->bhqk", q, k) * self.head_dim ** -0.5).softmax(-1)
        pooled = torch.einsum("bhqk,bkhd->bhqd", weights, v).transpose(1, 2).reshape(b, 1, -1)
        return (self.to_out(pooled) + start)[:, 0]


class _MLP(nn.Module):
    def __init__(self, hidden: int, ratio: float) -> None:
        super().__init__()
        self.norm = _RMSNorm(hidden)
        self.fc1 = nn.Linear(hidden, int(hidden * ratio))
        self.activation = nn.GELU()
        self.fc2 = nn.Linear(int(hidden * ratio), hidden)

    def forward(self, value: Tensor) -> Tensor:
        return value + self.fc2(self.activation(self.fc1(self.norm(value))))


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
        self.feature_layers = tuple(sorted(int(i) for i in feature_layers))
        if not self.feature_layers or len(set(self.feature_layers)) != len(self.feature_layers):
            raise ValueError(f"feature_layers must be unique and non-empty: {feature_layers}")
        if initial_logit_sign not in (-1.0, 1.0):
            raise ValueError("initial_logit_sign must be -1 or 1")
        self.initial_logit_sign = float(initial_logit_sign)
        self.seed = int(seed)
        with torch.device(init_device):
            self.branches = nn.ModuleList(_Branch(hidden_size, mlp_ratio, num_heads)
                                          for _ in self.feature_layers)
            width = hidden_size * len(self.feature_layers)
            self.final_norm = nn.LayerNorm(width, eps=1e-6)
            self.final_linear = nn.Linear(width, 1)
        if not any(p.is_meta for p in self.parameters()):
            self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, shard_index: int = 0) -> None:
        """Xavier-uniform linears, unit norms, N(0, 0.02) query tokens — from one seeded
        generator walked in module order."""
        generator = torch.Generator(device=self.final_linear.weight.device)
        generator.manual_seed(self.seed + int(shard_index))
        for module in self.modules():
            if isinstance(module, nn.Linear):
                fan_out, fan_in = module.weight.shape
                bound = (6.0 / float(fan_in + fan_out)) ** 0.5
                module.weight.uniform_(-bound, bound, generator=generator)
                if module.bias is not None:
                    module.bias.zero_()
            elif isinstance(module, (_RMSNorm, nn.LayerNorm)):
                module.weight.fill_(1.0)
                if getattr(module, "bias", None) is not None:
                    module.bias.zero_()
            elif isinstance(module, _QueryPool):
                module.query_token.normal_(0.0, 0.02, generator=generator)
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
