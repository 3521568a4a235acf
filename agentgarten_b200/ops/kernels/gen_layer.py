"""The two halves of a generation layer as fused inference calls.

``project(layer, hidden, cos, sin)``: RMSNorm → q/k/v GEMMs → per-head RMSNorm + RoPE.
``finish(layer, hidden, attention)``: output GEMM with the residual added in its epilogue →
RMSNorm → gate/up GEMMs → SiLU·mul → down GEMM with the residual in its epilogue.
Rounding follows the eager bf16 program (see ``csrc/pointwise.cu``).

Parity: reference ``wm/kernels/gen_layer.py:184-228``.
"""

from __future__ import annotations

import torch

from agentgarten_b200.ops import native

__all__ = ["finish", "project"]


def _native(layer, hidden: torch.Tensor) -> bool:
    return native.use(hidden) and layer.head_dim == 128 and layer.adaln is None


@torch.no_grad()
def project(layer, hidden: torch.Tensor, cosine: torch.Tensor, sine: torch.Tensor):
    if not _native(layer, hidden):
        return layer.project(hidden, cosine, sine)
    C = native.ext()
    b, n, h = hidden.shape
    to_q, to_k, to_v, _, norm_q, norm_k = layer.self_attn.parts()
    eps = layer.input_layernorm_moe_gen.variance_epsilon
    x2 = hidden.reshape(b * n, h)
    normed, _ = C.rms_norm_fwd(x2, layer.input_layernorm_moe_gen.weight, eps)
    gemm = lambda w: C.gemm(normed, w, False, True, None, False, None, None, torch.bfloat16)  # noqa: E731
    q, _ = C.head_norm_rope_fwd(gemm(to_q.weight).view(b, n, layer.num_attention_heads, 128),
                                norm_q.weight, cosine.contiguous(), sine.contiguous(), eps)
    k, _ = C.head_norm_rope_fwd(gemm(to_k.weight).view(b, n, layer.num_key_value_heads, 128),
                                norm_k.weight, cosine.contiguous(), sine.contiguous(), eps)
    v = gemm(to_v.weight).view(b, n, layer.num_key_value_heads, 128)
    native.count(6)
    return q, k, v


@torch.no_grad()
def finish(layer, hidden: torch.Tensor, attention: torch.Tensor) -> torch.Tensor:
    if not _native(layer, hidden):
        return layer.finish(hidden, attention)
    C = native.ext()
    b, n, h = hidden.shape
    mlp = layer.mlp_moe_gen
    eps = layer.post_attention_layernorm_moe_gen.variance_epsilon
    x2 = hidden.reshape(b * n, h)
    attn2 = attention.reshape(b * n, -1)
    bf16 = torch.bfloat16
    residual = C.gemm(attn2, layer.self_attn.parts()[3].weight, False, True, None, False, None, x2, bf16)
    normed, _ = C.rms_norm_fwd(residual, layer.post_attention_layernorm_moe_gen.weight, eps)
    act = C.silu_mul_fwd(C.gemm(normed, mlp.gate_proj.weight, False, True, None, False, None, None, bf16),
                         C.gemm(normed, mlp.up_proj.weight, False, True, None, False, None, None, bf16))
    out = C.gemm(act, mlp.down_proj.weight, False, True, None, False, None, residual, bf16)
    native.count(6)
    return out.view(b, n, h)
