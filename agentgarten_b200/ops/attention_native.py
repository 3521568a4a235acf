"""CUDA path of the attention operators (tcgen05 flash kernels, head_dim 128, bf16)."""

from __future__ import annotations

import torch

from . import native, reference
from .attention import AttentionSchedule, build_schedule

__all__ = ["dense", "jvp_dense", "planned"]


def _cat(chunks: list[torch.Tensor]) -> torch.Tensor:
    return chunks[0].contiguous() if len(chunks) == 1 else torch.cat(chunks, dim=1)


class _SegmentAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, text_k, text_v, text_valid, schedule: AttentionSchedule, scale):
        C = native.ext()
        out, lse = C.attn_fwd(q, k, v, text_k, text_v, text_valid, schedule.q_tiles,
                              schedule.entries, float(scale))
        native.count()
        ctx.save_for_backward(q, k, v, out, lse,
                              *(t for t in (text_k, text_v, text_valid) if t is not None))
        ctx.has_text = text_k is not None
        ctx.schedule, ctx.scale = schedule, float(scale)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        q, k, v, out, lse, *text = ctx.saved_tensors
        text_k, text_v, text_valid = text if ctx.has_text else (None, None, None)
        C = native.ext()
        dq, dk, dv = C.attn_bwd(grad.contiguous(), q, k, v, out, lse, text_k, text_v, text_valid,
                                ctx.schedule.q_tiles, ctx.schedule.entries,
                                ctx.schedule.k_tiles, ctx.schedule.q_lists, ctx.scale)
        native.count(3)
        return dq, dk, dv, None, None, None, None, None


def planned(queries, keys, values, plan, text_keys, text_values, text_valid):
    q = _cat(queries)
    k = _cat(keys)
    v = _cat(values)
    q_sizes = [c.shape[1] for c in queries]
    k_sizes = [c.shape[1] for c in keys]
    text_len = 0 if text_keys is None else int(text_keys.shape[1])
    schedule = build_schedule(q_sizes, k_sizes, plan, text_len, q.device)
    valid = None
    if text_keys is not None:
        valid = text_valid.to(device=q.device, dtype=torch.int32)
        text_keys, text_values = text_keys.contiguous(), text_values.contiguous()
    out = _SegmentAttention.apply(q, k, v, text_keys, text_values, valid, schedule,
                                  q.shape[-1] ** -0.5)
    return list(out.split(q_sizes, dim=1))


def dense(q, k, v, causal: bool = False):
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    schedule = build_schedule([q.shape[1]], [k.shape[1]], [[0]], 0, q.device, causal=causal)
    return _SegmentAttention.apply(q, k, v, None, None, None, schedule, q.shape[-1] ** -0.5)


def jvp_dense(q, k, v, dq, dk, dv, key_mask, prefix=None):
    """Primal and tangent on the tcgen05 JVP kernel.

    ``prefix = (text_len, text_valid)`` describes a key mask of the form "the first
    ``text_valid[b]`` of the first ``text_len`` keys, then everything"; any other mask goes
    to the FP64 PyTorch formula.  Tangents are rounded to bf16 like the primals.
    """
    C = native.ext()
    if key_mask is not None and prefix is None:
        o, do = reference.attention_jvp(q, k, v, dq, dk, dv, key_mask)
        return o.float(), do.float()
    native.count()
    text_len, text_valid = (0, None) if prefix is None else prefix
    if text_valid is not None:
        text_valid = text_valid.to(device=q.device, dtype=torch.int32).contiguous()
    bf16 = torch.bfloat16
    out, tangent, _ = C.attn_jvp(q.to(bf16).contiguous(), k.to(bf16).contiguous(), v.to(bf16).contiguous(),
                                 dq.to(bf16).contiguous(), dk.to(bf16).contiguous(), dv.to(bf16).contiguous(),
                                 q.shape[-1] ** -0.5, int(text_len), text_valid)
    return out, tangent
