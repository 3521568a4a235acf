"""Attention with forward-mode tangents: ``(O, dO)`` of softmax attention.

``attention_jvp(q, k, v, dq, dk, dv, key_mask=None, key_lengths=None)`` takes
``[B, H, N, D]`` tensors (the layout of ``scaled_dot_product_attention``) and returns FP32
``(O, dO)`` in the same layout.  ``backend_for`` names the implementation a call would
use: ``"tcgen05"`` (CUDA kernel of this package) or ``"reference"`` (FP64 PyTorch).

Parity: reference ``wm/kernels/attention_jvp/__init__.py:21-57`` (dispatch between CuTe and
Triton backends there).
"""

from __future__ import annotations

import torch

from agentgarten_b200 import ops
from agentgarten_b200.ops import native

__all__ = ["attention_jvp", "backend_for"]


def backend_for(q: torch.Tensor) -> str:
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and native.available() \
            and hasattr(native.ext(), "attn_jvp"):
        return "tcgen05"
    return "reference"


def attention_jvp(q, k, v, dq, dk, dv, *, key_mask=None, key_lengths=None):
    if key_lengths is not None:
        if key_mask is not None:
            raise ValueError("pass key_mask or key_lengths, not both")
        key_mask = torch.arange(k.shape[2], device=k.device)[None] < key_lengths[:, None]
    t = lambda x: x.transpose(1, 2)  # noqa: E731
    out, tangent = ops.attention_jvp(t(q), t(k), t(v), t(dq), t(dk), t(dv), key_mask)
    return t(out), t(tangent)
