"""Plain-PyTorch definitions of every operator in :mod:`agentgarten_b200.ops`.

These are the numerical oracles for the CUDA kernels and the implementation used on CPU
(and for dtypes the kernels do not cover).  Each function states the rounding points that
the kernels reproduce: statistics in at least FP32, a round to the activation dtype
wherever an eager bf16 program would store a tensor.

Parity: reference ``wm/networks/cosmos3/layers.py:67-170`` (RMSNorm, rotary),
``wm/networks/cosmos3/attention.py:56-83`` (attention and its FP64 JVP),
``wm/models/flow.py:49-59`` (rectified-flow pointwise), ``wm/kernels/stream_cache.py:16-54``
(cache relocation), ``wm/infra/optim/fused_adam.py:203-267`` (Adam math).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

__all__ = [
    "adam_update",
    "attention",
    "attention_jvp",
    "head_norm_rope",
    "linear",
    "relocate_rows",
    "rf_interpolate",
    "rf_x0",
    "rms_norm",
    "rms_norm_add",
    "rotate_half",
    "rotary",
    "silu_mul",
]


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    return F.linear(x, weight, bias)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``weight * round(x * rsqrt(mean(x^2) + eps))`` with FP32 (or wider) statistics."""
    wide = x.to(torch.promote_types(x.dtype, torch.float32))
    wide = wide * torch.rsqrt(wide.square().mean(-1, keepdim=True) + eps)
    return weight * wide.to(x.dtype)


def rms_norm_add(x: torch.Tensor, addend: torch.Tensor, weight: torch.Tensor, eps: float):
    """Residual add then RMSNorm; returns ``(x + addend, rms_norm(x + addend))``."""
    total = x + addend
    return total, rms_norm(total, weight, eps)


def rotate_half(value: torch.Tensor) -> torch.Tensor:
    first, second = value.chunk(2, dim=-1)
    return torch.cat((-second, first), dim=-1)


def rotary(value: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE. ``value`` is ``[B, N, H, D]``; tables are ``[B, N, D]``."""
    cos, sin = cos.unsqueeze(2), sin.unsqueeze(2)
    return value * cos + rotate_half(value) * sin


def head_norm_rope(value: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor,
                   sin: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head RMSNorm over ``D`` followed by RoPE."""
    return rotary(rms_norm(value, weight, eps), cos, sin)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


def rf_interpolate(x0: torch.Tensor, noise: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
    s = _broadcast_sigma(sigma.to(x0.dtype), x0)
    return (1.0 - s) * x0 + s * noise


def rf_x0(noisy: torch.Tensor, sigma: torch.Tensor, velocity: torch.Tensor) -> torch.Tensor:
    return noisy - _broadcast_sigma(sigma.to(noisy.dtype), noisy) * velocity


def _broadcast_sigma(sigma: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    # [B] → per sample; [B, T] → per frame of a [B, C, T, H, W] latent.
    if sigma.ndim == 1:
        return sigma.view(-1, *([1] * (like.ndim - 1)))
    return sigma[:, None, :, None, None]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              key_mask: torch.Tensor | None = None, causal: bool = False) -> torch.Tensor:
    """Softmax attention on ``[B, N, H, D]`` tensors with grouped KV heads.

    ``key_mask`` is ``[B, NK]`` boolean (True = visible).  Math in the input dtype through
    PyTorch SDPA, which accumulates in FP32.
    """
    mask = None if key_mask is None else key_mask[:, None, None, :]
    out = F.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
        attn_mask=mask, is_causal=causal, enable_gqa=q.shape[2] != k.shape[2])
    return out.transpose(1, 2)


def attention_jvp(q, k, v, dq, dk, dv, key_mask=None):
    """FP64 oracle: returns ``(O, dO)`` of softmax attention, ``[B, N, H, D]`` layout."""
    rep = q.shape[2] // k.shape[2]
    qd, dqd = (t.transpose(1, 2).double() for t in (q, dq))
    kd, vd, dkd, dvd = (t.transpose(1, 2).repeat_interleave(rep, 1).double() for t in (k, v, dk, dv))
    scale = q.shape[-1] ** -0.5
    s = qd @ kd.transpose(-1, -2) * scale
    if key_mask is not None:
        s = s.masked_fill(~key_mask[:, None, None, :], float("-inf"))
    p = s.softmax(-1)
    ds = (dqd @ kd.transpose(-1, -2) + qd @ dkd.transpose(-1, -2)) * scale
    dp = p * (ds - (p * ds).sum(-1, keepdim=True))
    return (p @ vd).transpose(1, 2), (dp @ vd + p @ dvd).transpose(1, 2)


def relocate_rows(rows: torch.Tensor, sink: int, shift: int, keep: int,
                  cos: torch.Tensor | None = None, sin: torch.Tensor | None = None) -> torch.Tensor:
    """FIFO eviction of a ``[N, H, D]`` cache: rows ``[sink, keep)`` take ``rows[r + shift]``.

    With ``cos``/``sin`` (``[keep - sink, D]`` FP32 rotation by the position delta) the moved
    rows are re-rotated with the rotate-half rule; values are moved without tables.
    """
    out = rows.clone()
    moved = rows[sink + shift: keep + shift]
    if cos is not None:
        wide = moved.float()
        wide = wide * cos[:, None, :] + rotate_half(wide) * sin[:, None, :]
        moved = wide.to(rows.dtype)
    out[sink:keep] = moved
    return out


def adam_update(param, grad, exp_avg, exp_avg_sq, master, *, lr, beta1, beta2, eps,
                weight_decay, step, adam_w_mode=True, grad_scale=1.0):
    """One Adam/AdamW step in FP32 on (optionally) master weights, in place.

    ``beta1 == 0`` skips the first moment (``exp_avg`` may be ``None``); ``beta2 == 0``
    uses ``|g|`` as the denominator.
    """
    g = grad.float() * grad_scale
    w = master if master is not None else param.float()
    if not adam_w_mode and weight_decay:
        g = g + weight_decay * w
    if beta1 > 0:
        exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
        m_hat = exp_avg / (1 - beta1 ** step)
    else:
        m_hat = g
    if beta2 > 0:
        exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        denom = (exp_avg_sq / (1 - beta2 ** step)).sqrt_().add_(eps)
    else:
        denom = g.abs().add_(eps)
    update = m_hat / denom
    if adam_w_mode and weight_decay:
        update = update + weight_decay * w
    w = w - lr * update
    if master is not None:
        master.copy_(w)
    param.copy_(w.to(param.dtype))
