"""Attention operators: dense, planned (segment lists) and forward-mode JVP.

``planned_attention`` is the single entry used by the attention policies.  A *plan* lists,
for every query chunk, the key/value chunks it may attend to; text keys (masked to each
sample's prompt length) always come first.  On a B200 the chunks are laid out back to back
and one flash kernel walks, per 128-row query tile, the list of key *segments* of its
chunk.  Key tiles never straddle segments, so the softmax of a query row is accumulated
over the same tile partition no matter how many other chunks are processed in the same
launch (bitwise replay between teacher-forced training and the cached rollout).

Parity: reference ``wm/networks/cosmos3/attention.py:56-217`` (SDPA per block with
concatenated keys and a boolean key mask; FP64 JVP oracle; autograd glue for tangents).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.autograd.forward_ad as fwAD

from . import native, reference

__all__ = ["AttentionSchedule", "attention", "attention_jvp", "build_schedule",
           "planned_attention"]

TILE = 128


def _has_tangent(*tensors: torch.Tensor) -> bool:
    return any(fwAD.unpack_dual(t).tangent is not None for t in tensors)


# --------------------------------------------------------------------------- JVP
def attention_jvp(q, k, v, dq, dk, dv, key_mask=None, prefix=None):
    """Primal and tangent of softmax attention, ``[B, N, H, D]`` layout → ``(O, dO)`` FP32.

    ``prefix = (text_len, text_valid)`` states that ``key_mask`` is a prefix-valid text
    segment followed by visible keys, the form the kernel masks by itself.
    """
    if native.use(q) and q.shape[-1] == 128:
        from .attention_native import jvp_dense

        return jvp_dense(q, k, v, dq, dk, dv, key_mask, prefix)
    o, do = reference.attention_jvp(q, k, v, dq, dk, dv, key_mask)
    return o.float(), do.float()


class _AttentionWithJVP(torch.autograd.Function):
    """Dense attention that also defines its forward-mode derivative."""

    @staticmethod
    def forward(q, k, v, key_mask, prefix):
        # a fresh contiguous tensor: forward-mode AD rejects outputs that are views
        return reference.attention(q, k, v, key_mask).contiguous()

    @staticmethod
    def setup_context(ctx, inputs, output):
        q, k, v, key_mask, prefix = inputs
        ctx.save_for_forward(q, k, v)
        ctx.save_for_backward(q, k, v)
        ctx.key_mask = key_mask
        ctx.prefix = prefix

    @staticmethod
    def backward(ctx, grad):
        q, k, v = ctx.saved_tensors
        with torch.enable_grad():
            q_, k_, v_ = (t.detach().requires_grad_(True) for t in (q, k, v))
            out = reference.attention(q_, k_, v_, ctx.key_mask)
            gq, gk, gv = torch.autograd.grad(out, (q_, k_, v_), grad)
        return gq, gk, gv, None, None

    @staticmethod
    def jvp(ctx, dq, dk, dv, _dmask, _dprefix):
        q, k, v = ctx.saved_tensors
        tangents = [torch.zeros_like(x) if dx is None else dx
                    for x, dx in ((q, dq), (k, dk), (v, dv))]
        _, tangent = attention_jvp(q, k, v, *tangents, key_mask=ctx.key_mask, prefix=ctx.prefix)
        return tangent.to(q.dtype).contiguous()


# ------------------------------------------------------------------------- dense
def attention(q, k, v, key_mask=None, causal: bool = False, prefix=None):
    """Softmax attention on ``[B, N, H, D]`` tensors with grouped KV heads.

    ``key_mask`` ``[B, NK]`` (True = visible); ``prefix = (text_len, text_valid)`` may state
    that it is a prefix-valid text segment followed by visible keys, which the tangent
    kernel masks by itself; arbitrary masks use the PyTorch path.
    """
    if _has_tangent(q, k, v):
        if causal:
            raise NotImplementedError("forward-mode causal attention is not used by any recipe")
        return _AttentionWithJVP.apply(q, k, v, key_mask, prefix)
    if native.use(q) and q.shape[-1] == 128 and key_mask is None:
        from .attention_native import dense

        return dense(q, k, v, causal=causal)
    return reference.attention(q, k, v, key_mask, causal)


# ----------------------------------------------------------------------- planned
@dataclass
class AttentionSchedule:
    """Device-side work lists for the segment flash kernels (all int32).

    ``q_tiles[t] = (q_row, rows, first_entry, entries, q_local)`` where ``q_local`` is the
    tile's first row counted from its chunk start; ``entries[e] = (source, k_row, k_len)``
    with source 0 = text (valid length per sample), 1 = visual, 2 = visual under a causal
    mask against the chunk.  ``k_tiles[t] = (k_row, rows, first_reader, readers, causal)``
    and ``q_lists[r] = (q_row, q_len)`` are the transposed lists used by the dK/dV pass.

    ``fused_tiles[t] = (k_row, rows, first_block, blocks, source)`` and ``fused_blocks[i] =
    (q_block_row, lo, hi, turn)`` describe the one-pass backward: key tiles (text tiles first,
    source 0) in the order in which they add to dQ, and for each tile the blocks of 128 query rows
    (aligned to multiples of 128) that see it, with the columns ``[lo, hi)`` of the block that
    do and the tile's turn among all tiles that add to that block.  None for causal schedules.
    """

    q_tiles: torch.Tensor
    entries: torch.Tensor
    k_tiles: torch.Tensor
    q_lists: torch.Tensor
    total_q: int
    total_k: int
    text_len: int
    fused_tiles: torch.Tensor | None = None
    fused_blocks: torch.Tensor | None = None


_schedule_cache: dict = {}


def build_schedule(q_sizes: list[int], k_sizes: list[int], plan: list[list[int]],
                   text_len: int, device: torch.device, causal: bool = False) -> AttentionSchedule:
    key = (tuple(q_sizes), tuple(k_sizes), tuple(map(tuple, plan)), text_len, str(device), causal)
    cached = _schedule_cache.get(key)
    if cached is not None:
        return cached
    k_start = [0]
    for size in k_sizes:
        k_start.append(k_start[-1] + size)
    q_tiles, entries = [], []
    q_row = 0
    readers: dict[int, list[tuple[int, int]]] = {j: [] for j in range(len(k_sizes))}
    for chunk, size in enumerate(q_sizes):
        first = len(entries)
        if text_len:
            entries.append((0, 0, text_len))
        for j in plan[chunk]:
            entries.append((2 if causal else 1, k_start[j], k_sizes[j]))
            readers[j].append((q_row, size))
        count = len(entries) - first
        for offset in range(0, size, TILE):
            q_tiles.append((q_row + offset, min(TILE, size - offset), first, count, offset))
        q_row += size
    k_tiles, q_lists = [], []
    for j, size in enumerate(k_sizes):
        first = len(q_lists)
        q_lists.extend(readers[j])
        count = len(q_lists) - first
        if count == 0:
            continue
        for offset in range(0, size, TILE):
            k_tiles.append((k_start[j] + offset, min(TILE, size - offset), first, count,
                            offset if causal else -1))

    def tensor(rows, width):
        data = torch.tensor(rows or [[0] * width], dtype=torch.int32).reshape(-1, width)
        return data.to(device)

    fused_tiles, fused_blocks = (None, None) if causal else _fused_lists(readers, k_sizes, k_start, text_len, q_row)
    schedule = AttentionSchedule(
        q_tiles=tensor(q_tiles, 5), entries=tensor(entries, 3), k_tiles=tensor(k_tiles, 5),
        q_lists=tensor(q_lists, 2), total_q=q_row, total_k=k_start[-1], text_len=text_len,
        fused_tiles=None if fused_tiles is None else tensor(fused_tiles, 5),
        fused_blocks=None if fused_blocks is None else tensor(fused_blocks, 4))
    if len(_schedule_cache) > 256:
        _schedule_cache.clear()
    _schedule_cache[key] = schedule
    return schedule


def _fused_lists(readers, k_sizes, k_start, text_len: int, total_q: int):
    """Work lists of the one-pass backward (see ``AttentionSchedule``)."""
    taken = [0] * (-(-total_q // TILE))          # turns handed out so far, per query block
    tiles, blocks = [], []

    def add_tile(k_row, rows, ranges, source):
        first = len(blocks)
        for q0, length in ranges:
            for block in range(q0 // TILE, (q0 + length - 1) // TILE + 1):
                lo = max(q0, block * TILE) - block * TILE
                hi = min(q0 + length, (block + 1) * TILE) - block * TILE
                blocks.append((block * TILE, lo, hi, taken[block]))
                taken[block] += 1
        if len(blocks) > first:
            tiles.append((k_row, rows, first, len(blocks) - first, source))

    def merged(ranges):
        out = []
        for q0, length in sorted(ranges):
            if out and out[-1][0] + out[-1][1] == q0:
                out[-1] = (out[-1][0], out[-1][1] + length)
            else:
                out.append((q0, length))
        return out

    if total_q == 0:
        return [], []
    for offset in range(0, text_len, TILE):
        add_tile(offset, min(TILE, text_len - offset), [(0, total_q)], 0)
    for j, size in enumerate(k_sizes):
        ranges = merged(readers[j])
        if not ranges:
            continue
        for offset in range(0, size, TILE):
            add_tile(k_start[j] + offset, min(TILE, size - offset), ranges, 1)
    return tiles, blocks


def _text_mask(text_valid, text_len: int, visual: int, device) -> torch.Tensor:
    valid = torch.arange(text_len, device=device)[None] < text_valid.to(device)[:, None]
    ones = torch.ones(valid.shape[0], visual, dtype=torch.bool, device=device)
    return torch.cat((valid, ones), dim=1)


def planned_attention(queries, keys, values, plan, *, text_keys=None, text_values=None,
                      text_valid=None):
    """Run a plan; returns one output per query chunk (``[B, N_c, H, D]``)."""
    q0 = queries[0]
    use_kernel = (native.use(q0) and q0.shape[-1] == 128
                  and not _has_tangent(*queries, *keys, *values))
    if use_kernel:
        from .attention_native import planned

        return planned(queries, keys, values, plan, text_keys, text_values, text_valid)
    text_len = 0 if text_keys is None else text_keys.shape[1]
    # Queries with identical key lists share one softmax call.
    groups: dict[tuple[int, ...], list[int]] = {}
    for index, visible in enumerate(plan):
        groups.setdefault(tuple(visible), []).append(index)
    outputs: list[torch.Tensor | None] = [None] * len(queries)
    for visible, members in groups.items():
        ks = [keys[j] for j in visible]
        vs = [values[j] for j in visible]
        if text_len:
            ks, vs = [text_keys, *ks], [text_values, *vs]
        key = torch.cat(ks, dim=1) if len(ks) > 1 else ks[0]
        value = torch.cat(vs, dim=1) if len(vs) > 1 else vs[0]
        mask, prefix = None, None
        if text_len:
            mask = _text_mask(text_valid, text_len, key.shape[1] - text_len, key.device)
            prefix = (text_len, text_valid)
        query = torch.cat([queries[i] for i in members], dim=1) if len(members) > 1 \
            else queries[members[0]]
        out = attention(query, key, value, mask, prefix=prefix)
        for i, piece in zip(members, out.split([queries[i].shape[1] for i in members], dim=1)):
            outputs[i] = piece
    return outputs
