"""CUDA path of the attention operators (tcgen05 flash kernels, head_dim 128, bf16)."""

from __future__ import annotations

import os

import torch

from . import native, reference
from .attention import AttentionSchedule, build_schedule

__all__ = ["dense", "jvp_dense", "planned"]


def _cat(chunks: list[torch.Tensor]) -> torch.Tensor:
    return chunks[0].contiguous() if len(chunks) == 1 else torch.cat(chunks, dim=1)


def segment_backward(C, grad, q, k, v, out, lse, text_k, text_v, text_valid, schedule, scale, dv_out):
    """(dq, dk, dv) of segment attention from the dQ and dK/dV kernels; ``AGB200_ATTN_BWD=fused``
    selects the one-pass kernel (``csrc/attention_bwd_fused.cu``) where the schedule has its work
    lists.  The one-pass form gives the same gradients bit-reproducibly but is the slower of the
    two today (6.2 against 3.5 ms at 8192 tokens), so it is not the default."""
    if schedule.fused_tiles is not None and os.environ.get("AGB200_ATTN_BWD", "split") == "fused":
        return C.attn_bwd_fused(grad, q, k, v, out, lse, text_k, text_v, text_valid,
                                schedule.fused_tiles, schedule.fused_blocks, scale, dv_out)
    return C.attn_bwd(grad, q, k, v, out, lse, text_k, text_v, text_valid, schedule.q_tiles,
                      schedule.entries, schedule.k_tiles, schedule.q_lists, scale, dv_out)


class _SegmentAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, text_k, text_v, text_valid, schedule: AttentionSchedule, scale):
        C = native.ext()
        out, lse = C.attn_fwd(q, k, v, text_k, text_v, text_valid, schedule.q_tiles,
                              schedule.entries, float(scale), 1)
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
        dq, dk, dv = segment_backward(C, grad.contiguous(), q, k, v, out, lse, text_k, text_v, text_valid,
                              ctx.schedule, ctx.scale, None)
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


_split_cache: dict = {}
_SM_COUNT: dict = {}


def _key_splits(batch: int, nq: int, nk: int, hq: int, hkv: int, device) -> int:
    """How many contiguous key ranges to run as separate CTAs so that the launch fills the GPU.

    The forward kernel has one CTA per (query tile, pair of heads, sample).  With few query
    tiles and many keys (a streamed block against its cache, a tensor-parallel shard) that is
    less than a wave of long-running CTAs; splitting the keys trades them for several waves of
    short ones.  Chooses the count that minimises waves x key tiles per CTA.
    """
    index = device.index if device.index is not None else torch.cuda.current_device()
    sms = _SM_COUNT.get(index)
    if sms is None:
        sms = _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
    heads_per_cta = 2 if (hq // hkv) % 2 == 0 else 1
    ctas = batch * -(-nq // 128) * (hq // heads_per_cta)
    tiles = -(-nk // 128)
    best, best_cost = 1, -(-ctas // sms) * tiles
    for splits in range(2, 9):
        per = -(-tiles // splits)
        if per < 8:  # too little work per CTA to amortise its prologue and the merge
            break
        cost = -(-(ctas * splits) // sms) * per + 2  # + the merge pass
        if cost < best_cost * 0.9:
            best, best_cost = splits, cost
    return best


def _split_schedule(nq: int, nk: int, splits: int, device):
    """Tile list with ``splits`` copies of the query tiles, copy ``s`` seeing key range ``s``."""
    key = (nq, nk, splits, str(device))
    hit = _split_cache.get(key)
    if hit is None:
        tiles = -(-nk // 128)
        per = -(-tiles // splits) * 128
        q_tiles, entries = [], []
        for s in range(splits):
            first = s * per
            entries.append((1, first, max(0, min(per, nk - first))))
            for offset in range(0, nq, 128):
                q_tiles.append((offset, min(128, nq - offset), s, 1, offset))
        hit = (torch.tensor(q_tiles, dtype=torch.int32, device=device),
               torch.tensor(entries, dtype=torch.int32, device=device))
        if len(_split_cache) > 256:
            _split_cache.clear()
        _split_cache[key] = hit
    return hit


def dense(q, k, v, causal: bool = False):
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if not causal and not needs_grad:
        splits = _key_splits(q.shape[0], q.shape[1], k.shape[1], q.shape[2], k.shape[2], q.device)
        if splits > 1:
            q_tiles, entries = _split_schedule(q.shape[1], k.shape[1], splits, q.device)
            native.count(2)
            out, _ = native.ext().attn_fwd(q, k, v, None, None, None, q_tiles, entries,
                                           q.shape[-1] ** -0.5, splits)
            return out
    if causal and needs_grad:
        # The dK/dV kernel has no per-element causal mask (the frozen text tower is the only
        # causal caller): a text tower that is being trained differentiates the PyTorch formula.
        return reference.attention(q, k, v, causal=True)
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
