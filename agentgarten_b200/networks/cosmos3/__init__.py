"""Cosmos3-Nano-shaped network family: layers, towers, attention policies, streaming.

``GEN_KEYS`` / ``TEXT_ENCODER_KEYS`` are the regular expressions that select the
generation-tower and text-tower tensors of the released transformer checkpoint.

Parity: reference ``wm/networks/cosmos3/__init__.py:16-68``.
"""

from __future__ import annotations

from dataclasses import asdict, is_dataclass
from typing import Any

import torch

from .layers import Cosmos3Config
from .network import Cosmos3Condition, Cosmos3Network, Cosmos3TextEncoder

__all__ = [
    "COSMOS3_EMPTY_PROMPT_IDS",
    "GEN_KEYS",
    "LORA_ATTENTION_MLP_MODULES",
    "LORA_ATTENTION_MODULES",
    "TEXT_ENCODER_KEYS",
    "Cosmos3Condition",
    "Cosmos3Conditioner",
    "Cosmos3Config",
    "Cosmos3Network",
    "Cosmos3TextEncoder",
    "build_network",
]

# The patterns end up verbatim in resolved configuration files (``source_model_key_patterns``),
# so they are spelled exactly as the reference spells them.
TEXT_ENCODER_KEYS = (
    r"embed_tokens\.weight",
    r"layers\.\d+\.self_attn\.(?:to_q|to_k|to_v|to_out|norm_q|norm_k)\.weight",
    r"layers\.\d+\.(?:input_layernorm|post_attention_layernorm)\.weight",
    r"layers\.\d+\.mlp\.(?:gate|up|down)_proj\.weight",
)
GEN_KEYS = (
    r"layers\.\d+\.self_attn\.(?:add_[qkv]_proj|to_add_out|norm_added_[qk])\.weight",
    r"layers\.\d+\.(?:input_layernorm_moe_gen|post_attention_layernorm_moe_gen)\.weight",
    r"layers\.\d+\.mlp_moe_gen\.(?:gate|up|down)_proj\.weight",
    r"norm_moe_gen\.weight",
    r"proj_(?:in|out)\.(?:weight|bias)",
    r"time_embedder\.linear_[12]\.(?:weight|bias)",
    r"geometry_modality_embed",       # trained checkpoints only; absent from the released one
    r"first_frame_reference_embed",
)
LORA_ATTENTION_MODULES = (r"layers\.\d+\.self_attn\.(?:add_[qkv]_proj|to_add_out)",)
LORA_ATTENTION_MLP_MODULES = (
    *LORA_ATTENTION_MODULES,
    r"layers\.\d+\.mlp_moe_gen\.(?:gate|up|down)_proj",
)
# Token ids of an empty user message after the chat template (text dropout / default negative).
COSMOS3_EMPTY_PROMPT_IDS: tuple[int, ...] = (151644, 872, 198, 151645, 198, 151644, 77091, 198)


def _as_config(config: Any) -> Cosmos3Config:
    if isinstance(config, Cosmos3Config):
        return config
    if is_dataclass(config):
        return Cosmos3Config(**asdict(config))
    data = {k: v for k, v in dict(config).items() if not str(k).startswith("_")}
    return Cosmos3Config(**data)


def build_network(config: Any, *, init_device: str | torch.device = "meta",
                  lora: dict | None = None) -> Cosmos3Network:
    """Construct the generation tower on ``init_device`` and optionally inject LoRA."""
    with torch.device(init_device):
        network = Cosmos3Network(_as_config(config))
    if lora:
        from agentgarten_b200.networks.lora import inject_lora

        inject_lora(network, lora)
    return network


def __getattr__(name: str):
    if name == "Cosmos3Conditioner":
        from .conditioner import Cosmos3Conditioner

        return Cosmos3Conditioner
    raise AttributeError(name)
