"""Low-rank adapters for linear layers.

``inject_lora`` swaps every matching linear (by regex full match on any of its module
names) for a :class:`LoRALinear` that shares the original weight tensor.  The adapter adds
``B(A(dropout(x))) * alpha / rank``; ``B`` starts at zero so injection is a no-op until
training moves it.  Initialisation is seeded and runs in module-traversal order, so every
rank builds identical adapters.

Parity: reference ``wm/networks/lora.py:13-182``.
"""

from __future__ import annotations

import math
import re
from collections.abc import Mapping
from typing import Any

import torch
from torch import nn

from agentgarten_b200 import ops

__all__ = ["LORA_PARAMETER_PATTERN", "LoRALinear", "initialize_lora_parameters", "inject_lora"]

LORA_PARAMETER_PATTERN = r"(?:.+\.)?lora_[AB]\.weight"


class LoRALinear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, rank: int,
                 alpha: float, dropout: float = 0.0, device=None, dtype=None) -> None:
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self._attach(rank, alpha, dropout, device, dtype)

    def _attach(self, rank: int, alpha: float, dropout: float, device, dtype) -> None:
        self.rank, self.alpha = int(rank), float(alpha)
        self.scaling = self.alpha / self.rank
        self.lora_dropout = nn.Dropout(float(dropout)) if dropout else nn.Identity()
        self.lora_A = nn.Linear(self.in_features, self.rank, bias=False, device=device, dtype=dtype)
        self.lora_B = nn.Linear(self.rank, self.out_features, bias=False, device=device, dtype=dtype)
        self.reset_lora_parameters()

    @classmethod
    def from_linear(cls, linear: nn.Linear, *, rank: int, alpha: float, dropout: float):
        """Wrap an existing linear without allocating a second base weight."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.weight = linear.weight
        if linear.bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = linear.bias
        self._attach(rank, alpha, dropout, linear.weight.device, linear.weight.dtype)
        self.train(linear.training)
        return self

    @torch.no_grad()
    def reset_lora_parameters(self) -> None:
        if self.lora_A.weight.is_meta:
            return
        nn.init.kaiming_uniform_(self.lora_A.weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B.weight)

    def forward(self, input: torch.Tensor) -> torch.Tensor:  # noqa: A002 (nn.Linear's name)
        base = ops.linear(input, self.weight, self.bias)
        low = ops.linear(self.lora_dropout(input), self.lora_A.weight)
        return base + ops.linear(low, self.lora_B.weight) * self.scaling


def inject_lora(module: nn.Module, config: Mapping[str, Any] | None) -> tuple[str, ...]:
    """Replace matching linears; returns the sorted names that were replaced."""
    if config is None:
        return ()
    rank = int(config.get("rank", 16))
    alpha = float(config.get("alpha", rank))
    dropout = float(config.get("dropout", 0.0))
    patterns = config.get("module_patterns", ())
    patterns = (patterns,) if isinstance(patterns, str) else tuple(patterns)
    if rank <= 0:
        raise ValueError("LoRA rank must be positive")
    if not 0.0 <= dropout < 1.0:
        raise ValueError("LoRA dropout must be in [0, 1)")
    compiled = [re.compile(p) for p in patterns]
    if not compiled:
        return ()
    names_of: dict[int, list[str]] = {}
    module_of: dict[int, nn.Linear] = {}
    for name, child in module.named_modules(remove_duplicate=False):
        if name and isinstance(child, nn.Linear) and not isinstance(child, LoRALinear) \
                and not name.rsplit(".", 1)[-1].startswith("lora_"):
            names_of.setdefault(id(child), []).append(name)
            module_of[id(child)] = child
    replaced: list[str] = []
    # dict order == traversal order, so RNG use is the same on every rank.
    for identity, names in names_of.items():
        if not any(c.fullmatch(n) for n in names for c in compiled):
            continue
        adapter = LoRALinear.from_linear(module_of[identity], rank=rank, alpha=alpha, dropout=dropout)
        for name in names:
            parent_name, _, leaf = name.rpartition(".")
            parent = module.get_submodule(parent_name) if parent_name else module
            parent._modules[leaf] = adapter
            replaced.append(name)
    return tuple(sorted(replaced))


@torch.no_grad()
def initialize_lora_parameters(module: nn.Module, seed: int = 0) -> None:
    """Seeded re-initialisation of every adapter (after meta materialisation)."""
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(seed)
        for child in module.modules():
            if isinstance(child, LoRALinear):
                child.reset_lora_parameters()
