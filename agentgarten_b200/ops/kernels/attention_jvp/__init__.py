"""Attention with forward-mode tangents: ``(O, dO)`` of softmax attention.

``attention_jvp(q, k, v, dq, dk, dv, key_mask=None, scale=None, backend=None)`` takes
``[B, H, N, D]`` tensors (the layout of ``scaled_dot_product_attention``) and returns FP32
``(O, dO)`` in the same layout.  ``backend_for`` names the implementation a call would
use: ``"tcgen05"`` (CUDA kernel of this package) or ``"reference"`` (FP64 PyTorch).

Parity: reference ``wm/kernels/attention_jvp/__init__.py:21-57`` (dispatch between CuTe and
Triton backends there; the names of those backends are not accepted here).
"""

from __future__ import annotations

import torch

from agentgarten_b200 import ops
from agentgarten_b200.ops import native

__all__ = ["attention_jvp", "backend_for"]

_BACKENDS = ("tcgen05", "reference")


def backend_for(device) -> str:
    """The implementation used on ``device`` (a device, or a query tensor: dtype and head size
    then count as well, since the kernel takes bf16 heads of 128)."""
    if torch.is_tensor(device):
        q = device
        fits = q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128
    else:
        fits = torch.device(device).type == "cuda"
    if fits and native.available() and hasattr(native.ext(), "attn_jvp"):
        return "tcgen05"
    return "reference"


@torch.no_grad()
def attention_jvp(q, k, v, dq, dk, dv, *, key_mask=None, scale=None, backend=None, key_lengths=None):
    if backend is not None and backend not in _BACKENDS:
        raise ValueError(f"attention_jvp backend must be one of {_BACKENDS}, got {backend!r}")
    if key_lengths is not None:
        if key_mask is not None:
            raise ValueError("pass key_mask or key_lengths, not both")
        key_mask = torch.arange(k.shape[2], device=k.device)[None] < key_lengths[:, None]
    if scale is not None:
        # the operators use head_dim ** -0.5; any other scale is folded into the query side
        factor = float(scale) / float(q.shape[-1]) ** -0.5
        if factor != 1.0:
            q, dq = q * factor, dq * factor
    t = lambda x: x.transpose(1, 2)  # noqa: E731
    if backend == "reference":
        from agentgarten_b200.ops import reference

        out, tangent = reference.attention_jvp(t(q), t(k), t(v), t(dq), t(dk), t(dv), key_mask)
        return t(out).float(), t(tangent).float()
    out, tangent = ops.attention_jvp(t(q), t(k), t(v), t(dq), t(dk), t(dv), key_mask)
    return t(out), t(tangent)
