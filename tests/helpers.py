"""Shared builders for tests: a tiny DiT, a tiny conditioner and synthetic batches."""

import torch

from agentgarten_b200.networks.cosmos3 import Cosmos3Config, build_network
from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner


def tiny_config(**overrides):
    base = dict(hidden_size=256, intermediate_size=1024, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=128,
                mrope_section=(12, 10, 10), text_bucket_tokens=16,
                special_tokens={"eos_token_id": 1, "start_of_generation": 2})
    base.update(overrides)
    return Cosmos3Config(**base)


def tiny_network(config=None, device="cpu", dtype=torch.float32, seed=0):
    config = config or tiny_config()
    torch.manual_seed(seed)
    net = build_network(config, init_device=device).to(dtype)
    with torch.no_grad():
        for p in net.parameters():
            if p.ndim >= 2:
                torch.nn.init.normal_(p, std=0.02)
        net.geometry_modality_embed.normal_(std=0.02)
        net.first_frame_reference_embed.normal_(std=0.02)
    return net


def tiny_conditioner(config=None, device="cpu", dtype=torch.float32, seed=1):
    config = config or tiny_config()
    torch.manual_seed(seed)
    cond = Cosmos3Conditioner(config=config, codec=None, init_device=device,
                              geometry_noise_sigma=0.0)
    cond.to(dtype)
    with torch.no_grad():
        for p in cond.parameters():
            if p.ndim >= 2:
                torch.nn.init.normal_(p, std=0.02)
    return cond


def synthetic_batch(batch=1, frames=5, height=8, width=8, channels=48, text=10, vocab=128,
                    device="cpu", seed=0, geometry_hw=None):
    g = torch.Generator().manual_seed(seed)
    gh, gw = geometry_hw or (height, width)
    return {
        "latent": torch.randn(batch, channels, frames, height, width, generator=g).to(device),
        "depth_latent": torch.randn(batch, channels, frames, gh, gw, generator=g).to(device),
        "normal_latent": torch.randn(batch, channels, frames, gh, gw, generator=g).to(device),
        "text_input_ids": torch.randint(3, vocab, (batch, text), generator=g).to(device),
        "fps": torch.full((batch,), 16.0).to(device),
    }
