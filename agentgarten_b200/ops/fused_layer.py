"""Whole-layer execution of a generation layer on the CUDA kernels, with a hand-written
backward.

All chunks of a step are concatenated along tokens and pushed through the layer as one
matrix (the GEMM and every row kernel are row-invariant, so per-row results equal those of
chunk-by-chunk execution).  The forward keeps only the layer input, the attention output
and its log-sum-exp; the backward recomputes the cheap parts (norms, projections, MLP
activations) and runs the tcgen05 GEMMs for input and weight gradients, accumulating
weight gradients straight into the parameters' ``.grad`` buffers (fp32-accumulated in
TMEM, no temporary per microbatch).  This is the "selective" activation policy: attention
outputs are kept, everything else is recomputed.

Parity: reference ``wm/networks/cosmos3/layers.py:269-312`` (project / finish) run under
``wm/infra/parallel.py:164-214`` (selective activation checkpointing).

The q, k and v projections run as one GEMM (N = q + 2 kv widths) and gate and up as another
whenever their weight matrices lie back to back in one storage, which is how the optimizer
engine's flat parameter buffer lays them out (``parallel/zero.py``); their gradient buffers
are adjacent in the same way, so each group also takes one input-gradient and one
weight-gradient GEMM in the backward pass.  The head norm reads q and k as column slices of
the joint product, attention reads v as one, and the attention backward writes dv straight
into the v columns of the joint gradient.  Weights that are not adjacent (a model without the
flat buffer) take one GEMM each; an output column is the same K-ordered sum either way.

Recomputation is a memory policy, not a numerical one: when the device has room, a layer
keeps the activations of its MLP half (``h1``, its norm, gate, up: 65 KB per token) and of
its attention half (``n1``, q/k/v before and after the head norm: 31 KB per token) and the
backward skips the corresponding GEMMs.  The decision is taken per layer at forward time
from the free device memory minus a reserve, so a 7 B model on one 180 GB GPU recomputes
almost everything while the same job with the optimizer state sharded over several GPUs
recomputes nothing.  Results are bitwise identical either way (same kernels, same inputs).
"""

from __future__ import annotations

import os

import torch

from agentgarten_b200.utils.trace import span

from . import native
from .attention import build_schedule
from .linear import joined as _joined
from .attention_native import segment_backward as attention_backward

__all__ = ["eligible", "keep_policy", "run"]

# Free device memory that is never spent on kept activations (backward workspaces, optimizer
# temporaries, allocator fragmentation), and an optional hard switch.
_RESERVE_BYTES = int(float(os.environ.get("AGB200_ACTIVATION_RESERVE_GB", "12")) * (1 << 30))
_KEEP_MODE = os.environ.get("AGB200_KEEP_ACTIVATIONS", "auto")  # auto | never | always


def keep_policy(tokens: int, hidden: int, inner: int, q_width: int, kv_width: int,
                device: torch.device, layers_ahead: int = 0) -> tuple[bool, bool]:
    """(keep MLP half, keep attention half) for one layer about to run its forward.

    ``layers_ahead`` layers still have to run after this one in the same pass; each of them saves
    at least its input and its attention output, and that memory is set aside before anything
    optional is kept (a long clip on one GPU would otherwise spend it here and run out there)."""
    if _KEEP_MODE == "never":
        return False, False
    if _KEEP_MODE == "always":
        return True, True
    free, _ = torch.cuda.mem_get_info(device)
    free += torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    free -= layers_ahead * tokens * (hidden + q_width) * 2
    free -= tokens * 65536   # the backward pass of a layer needs workspace in proportion to its rows
    mlp_bytes = tokens * (2 * hidden + 2 * inner) * 2
    attn_bytes = tokens * (hidden + 2 * q_width + 3 * kv_width) * 2
    keep_mlp = free - mlp_bytes > _RESERVE_BYTES
    keep_attn = keep_mlp and free - mlp_bytes - attn_bytes > _RESERVE_BYTES
    return keep_mlp, keep_attn


def _plain_linear(module) -> bool:
    from agentgarten_b200.networks.lora import LoRALinear

    return (isinstance(module, torch.nn.Linear) and not isinstance(module, LoRALinear)
            and module.bias is None)


def eligible(layer, chunks, attention=None) -> bool:
    import os

    if os.environ.get("AGB200_DISABLE_FUSED_LAYER") == "1":
        return False
    first = chunks[0]
    if not (first.is_cuda and first.dtype == torch.bfloat16 and torch.is_grad_enabled()):
        return False
    if not native.available() or layer.head_dim != 128 or layer.adaln is not None:
        return False
    if attention is not None and not hasattr(attention, "plan"):
        return False
    attn, mlp = layer.self_attn, layer.mlp_moe_gen
    linears = [*attn.parts()[:4], mlp.gate_proj, mlp.up_proj, mlp.down_proj]
    if not all(_plain_linear(m) for m in linears):
        return False
    import torch.autograd.forward_ad as fwAD

    return fwAD.unpack_dual(first).tangent is None


def _gemm(a, w, **kw):
    C = native.ext()
    native.count()
    return C.gemm(a, w, kw.get("trans_a", False), kw.get("trans_b", True), kw.get("out"),
                  kw.get("accumulate", False), None, kw.get("residual"), torch.bfloat16)


def _wgrad(weight: torch.Tensor, grad_rows: torch.Tensor, input_rows: torch.Tensor):
    """dW[N, K] (+)= grad_rows[M, N]^T @ input_rows[M, K]; returns a tensor only when the
    parameter has no gradient buffer yet."""
    if not weight.requires_grad:
        return None
    if weight.grad is not None:
        _gemm(grad_rows, input_rows, trans_a=True, trans_b=False, out=weight.grad, accumulate=True)
        return None
    return _gemm(grad_rows, input_rows, trans_a=True, trans_b=False)


def _wgrad_group(weights, grad_rows: torch.Tensor, input_rows: torch.Tensor):
    """Weight gradients of matrices whose products were computed as one GEMM: ``grad_rows`` holds
    their output gradients side by side.  One GEMM into the joint gradient buffer when the
    buffers are adjacent, else one per matrix from the column slices."""
    joint = _joined([w.grad if w.requires_grad else None for w in weights])
    if joint is not None:
        _gemm(grad_rows, input_rows, trans_a=True, trans_b=False, out=joint, accumulate=True)
        return [None] * len(weights)
    results, at = [], 0
    for w in weights:
        results.append(_wgrad(w, grad_rows[:, at:at + w.shape[0]], input_rows))
        at += w.shape[0]
    return results


def _project_qkv(C, n1, weights, shape, cos, sin, eps):
    """(q_lin, k_lin, q, k, v, rstd_q, rstd_k, joint): the three projections of the normalised
    rows and the head norm + RoPE of q and k.  ``joint`` is the [rows, q | k | v] product when one
    GEMM made it (q_lin, k_lin and v are then column slices of it), else None."""
    b, n, heads, kv_heads = shape
    wq, wk, wv, nq, nk = weights
    wqkv = _joined((wq, wk, wv))
    if wqkv is not None:
        joint = _gemm(n1, wqkv).view(b, n, -1)
        q_lin = joint[..., :heads * 128].unflatten(-1, (heads, 128))
        k_lin = joint[..., heads * 128:(heads + kv_heads) * 128].unflatten(-1, (kv_heads, 128))
        v = joint[..., (heads + kv_heads) * 128:].unflatten(-1, (kv_heads, 128))
    else:
        joint = None
        q_lin = _gemm(n1, wq).view(b, n, heads, 128)
        k_lin = _gemm(n1, wk).view(b, n, kv_heads, 128)
        v = _gemm(n1, wv).view(b, n, kv_heads, 128)
    q, rq = C.head_norm_rope_fwd(q_lin, nq, cos, sin, eps)
    k, rk = C.head_norm_rope_fwd(k_lin, nk, cos, sin, eps)
    return q_lin, k_lin, q, k, v, rq, rk, joint


def _gate_up(C, n2, wg, wu, activation: bool = True):
    """(activation, kept): silu(gate) * up of the normalised rows; ``kept`` is what the backward
    needs of the projections: the joint [rows, gate | up] product, or the pair.  With
    ``activation=False`` the joint form leaves the activation to the caller (the backward pass
    gets it from the kernel that also produces the gradient of the product)."""
    wgu = _joined((wg, wu))
    if wgu is not None:
        both = _gemm(n2, wgu)
        return (C.silu_mul_pair(both) if activation else None), (both,)
    gate, up = _gemm(n2, wg), _gemm(n2, wu)
    return C.silu_mul_fwd(gate, up), (gate, up)


class _Layer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, layer, schedule, text_k, text_v, text_valid, layers_ahead, *weights):
        C = native.ext()
        w_in, wq, wk, wv, wo, nq, nk, w_post, wg, wu, wd = weights
        b, n, h = x.shape
        eps, heads, kv_heads = layer.input_layernorm_moe_gen.variance_epsilon, \
            layer.num_attention_heads, layer.num_key_value_heads
        x2 = x.reshape(b * n, h)
        keep_mlp, keep_attn = keep_policy(b * n, h, wg.shape[0], wq.shape[0], wk.shape[0], x.device,
                                          layers_ahead)
        n1, rstd1 = C.rms_norm_fwd(x2, w_in, eps)
        q_lin, k_lin, q, k, v, rq, rk, _ = _project_qkv(C, n1, (wq, wk, wv, nq, nk),
                                                        (b, n, heads, kv_heads), cos, sin, eps)
        attn, lse = C.attn_fwd(q, k, v, text_k, text_v, text_valid, schedule.q_tiles,
                               schedule.entries, 128 ** -0.5, 1)
        h1 = _gemm(attn.view(b * n, heads * 128), wo, residual=x2)
        n2, rstd2 = C.rms_norm_fwd(h1, w_post, eps)
        act, projected = _gate_up(C, n2, wg, wu)
        y = _gemm(act, wd, residual=h1)
        native.count(7)
        ctx.layer, ctx.schedule = layer, schedule
        ctx.text = (text_k, text_v, text_valid)
        ctx.params = weights  # the parameter objects themselves (their .grad buffers are used)
        ctx.kept_mlp = (h1, n2, rstd2, projected) if keep_mlp else None
        ctx.kept_attn = (n1, rstd1, q_lin, k_lin, q, k, v, rq, rk) if keep_attn else None
        ctx.save_for_backward(x, cos, sin, attn, lse, *weights)
        if any(w.requires_grad for w in weights):
            from agentgarten_b200.parallel import zero

            zero.note_forward(weights)  # its backward reports the layer's gradients to the optimizer engine
        return y.view(b, n, h)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        with span("layer backward"):
            return _Layer._backward(ctx, dy)

    @staticmethod
    def _backward(ctx, dy):
        C = native.ext()
        x, cos, sin, attn, lse, *_ = ctx.saved_tensors
        w_in, wq, wk, wv, wo, nq, nk, w_post, wg, wu, wd = ctx.params
        layer, schedule = ctx.layer, ctx.schedule
        text_k, text_v, text_valid = ctx.text
        b, n, h = x.shape
        eps, heads, kv_heads = layer.input_layernorm_moe_gen.variance_epsilon, \
            layer.num_attention_heads, layer.num_key_value_heads
        x2 = x.reshape(b * n, h)
        dy2 = dy.reshape(b * n, h).contiguous()
        attn2 = attn.view(b * n, heads * 128)
        # ---- the second half: kept, or recomputed
        if ctx.kept_mlp is not None:
            h1, n2, rstd2, projected = ctx.kept_mlp
            ctx.kept_mlp = None
            act = None if len(projected) == 1 else C.silu_mul_fwd(*projected)
        else:
            h1 = _gemm(attn2, wo, residual=x2)
            n2, rstd2 = C.rms_norm_fwd(h1, w_post, eps)
            act, projected = _gate_up(C, n2, wg, wu, activation=False)
        # ---- MLP backward
        dact = _gemm(dy2, wd, trans_b=False)
        if len(projected) == 1:   # gate | up came from one GEMM: one GEMM each way back as well
            # one pass over the product gives its gradient and the activation the down projection's
            # weight gradient needs
            dboth, act = C.silu_mul_pair_bwd_act(dact, projected[0])
            del dact, projected
            dwd = _wgrad(wd, dy2, act)
            del act
            dwg, dwu = _wgrad_group((wg, wu), dboth, n2)
            dn2 = _gemm(dboth, _joined((wg, wu)), trans_b=False)
            del dboth, n2
        else:
            dwd = _wgrad(wd, dy2, act)
            del act
            dgate, dup = C.silu_mul_bwd(dact, *projected)
            del dact, projected
            dwg, dwu = _wgrad(wg, dgate, n2), _wgrad(wu, dup, n2)
            dn2 = _gemm(dgate, wg, trans_b=False)
            _gemm(dup, wu, trans_b=False, out=dn2, accumulate=True)
            del dgate, dup, n2
        dh1, dw_post = C.rms_norm_bwd_add(dn2, h1, w_post, rstd2, dy2)   # + the residual branch
        del dn2, h1
        # ---- output projection backward
        dwo = _wgrad(wo, dh1, attn2)
        dattn = _gemm(dh1, wo, trans_b=False).view(b, n, heads, 128)
        # ---- the first half: kept, or recomputed
        if ctx.kept_attn is not None:
            n1, rstd1, q_lin, k_lin, q, k, v, rq, rk = ctx.kept_attn
            ctx.kept_attn = None
        else:
            n1, rstd1 = C.rms_norm_fwd(x2, w_in, eps)
            q_lin, k_lin, q, k, v, rq, rk, _ = _project_qkv(C, n1, (wq, wk, wv, nq, nk),
                                                            (b, n, heads, kv_heads), cos, sin, eps)
        wqkv = _joined((wq, wk, wv))
        if wqkv is not None:
            # One [rows, q | k | v] gradient: attention writes dv into its columns, the head-norm
            # backward writes dq and dk into theirs; then one GEMM each for dW and dx.
            split = (heads * 128, (heads + kv_heads) * 128)
            dqkv = torch.empty(b, n, wqkv.shape[0], device=x.device, dtype=x.dtype)
            dv = dqkv[..., split[1]:].unflatten(-1, (kv_heads, 128))
            dv.zero_()
            dq, dk, _ = attention_backward(C, dattn, q, k, v, attn, lse, text_k, text_v, text_valid,
                                           schedule, 128 ** -0.5, dv)
            del dattn, q, k, v
            _, dnq = C.head_norm_rope_bwd(dq, q_lin, nq, cos, sin, rq,
                                          dqkv[..., :split[0]].unflatten(-1, (heads, 128)))
            _, dnk = C.head_norm_rope_bwd(dk, k_lin, nk, cos, sin, rk,
                                          dqkv[..., split[0]:split[1]].unflatten(-1, (kv_heads, 128)))
            del dq, dk, q_lin, k_lin
            dqkv = dqkv.view(b * n, -1)
            dwq, dwk, dwv = _wgrad_group((wq, wk, wv), dqkv, n1)
            dn1 = _gemm(dqkv, wqkv, trans_b=False)
            del dqkv
        else:
            dq, dk, dv = attention_backward(C, dattn, q, k, v, attn, lse, text_k, text_v, text_valid,
                                            schedule, 128 ** -0.5, None)
            del dattn, q, k, v
            dq_lin, dnq = C.head_norm_rope_bwd(dq, q_lin, nq, cos, sin, rq, None)
            dk_lin, dnk = C.head_norm_rope_bwd(dk, k_lin, nk, cos, sin, rk, None)
            del dq, dk, q_lin, k_lin
            dq2, dk2, dv2 = dq_lin.view(b * n, -1), dk_lin.view(b * n, -1), dv.view(b * n, -1)
            dwq, dwk, dwv = _wgrad(wq, dq2, n1), _wgrad(wk, dk2, n1), _wgrad(wv, dv2, n1)
            dn1 = _gemm(dq2, wq, trans_b=False)
            _gemm(dk2, wk, trans_b=False, out=dn1, accumulate=True)
            _gemm(dv2, wv, trans_b=False, out=dn1, accumulate=True)
        dx, dw_in = C.rms_norm_bwd_add(dn1, x2, w_in, rstd1, dh1)        # + the residual branch
        native.count(20)
        # Vector gradients go into the parameters' gradient buffers here as well (autograd would
        # only add returned values after this function), so that the layer can be reported to
        # the optimizer engine as complete: its bucket is then reduced over the peers while the
        # backward pass of the earlier layers runs.
        dw_in, dnq, dnk, dw_post = (_accumulate(w, g) for w, g in
                                    ((w_in, dw_in), (nq, dnq), (nk, dnk), (w_post, dw_post)))
        if any(w.requires_grad for w in ctx.params):
            from agentgarten_b200.parallel import zero

            zero.grads_ready(ctx.params)
        return (dx.view(b, n, h), None, None, None, None, None, None, None, None,
                dw_in, dwq, dwk, dwv, dwo, dnq, dnk, dw_post, dwg, dwu, dwd)


def _accumulate(weight: torch.Tensor, grad):
    """Add ``grad`` to an existing gradient buffer of ``weight`` (returns None), or hand it to
    autograd in the parameter's dtype when there is none yet."""
    if grad is None or not weight.requires_grad:
        return None
    if weight.grad is not None:
        weight.grad.add_(grad.to(weight.grad.dtype))
        return None
    return grad.to(weight.dtype)


_rope_cache: tuple | None = None   # (ids of the per-chunk tables, the tables, their concatenations)


def _joined_ropes(ropes):
    """The per-chunk cos / sin tables as one table each; the same list comes back for every layer
    of a pass, so the concatenation is made once per pass."""
    global _rope_cache
    if len(ropes) == 1:
        return ropes[0]
    key = tuple(id(t) for pair in ropes for t in pair)
    if _rope_cache is None or _rope_cache[0] != key:
        cos = torch.cat([r[0] for r in ropes], dim=1)
        sin = torch.cat([r[1] for r in ropes], dim=1)
        _rope_cache = (key, list(ropes), (cos, sin))   # the sources are kept so that their ids stay theirs
    return _rope_cache[2]


def _whole_of(chunks, sizes):
    """The tensor these chunks were split from by the previous layer's :func:`run`, when they are
    exactly its pieces in order; else None.  Using it skips a concatenation per layer (and, in
    the backward pass, the concatenation of the pieces' gradients)."""
    whole = getattr(chunks[0], "_agb_whole", None)
    if whole is None or getattr(whole, "_agb_sizes", None) != tuple(sizes):
        return None
    for index, chunk in enumerate(chunks):
        if getattr(chunk, "_agb_whole", None) is not whole or getattr(chunk, "_agb_index", -1) != index:
            return None
    return whole


def run(layer, chunks, ropes, attention, layer_index):
    sizes = [c.shape[1] for c in chunks]
    if len(chunks) == 1:
        x = chunks[0]
    else:
        x = _whole_of(chunks, sizes)
        if x is None:
            x = torch.cat(chunks, dim=1)
    cos, sin = _joined_ropes(ropes)
    plan = attention.plan(len(chunks))
    text = attention.text
    text_k, text_v = text.keys[layer_index].contiguous(), text.values[layer_index].contiguous()
    valid = text.valid_lengths.to(device=x.device, dtype=torch.int32)
    schedule = build_schedule(sizes, sizes, plan, int(text_k.shape[1]), x.device)
    attn, mlp = layer.self_attn, layer.mlp_moe_gen
    to_q, to_k, to_v, to_out, norm_q, norm_k = attn.parts()
    weights = (layer.input_layernorm_moe_gen.weight, to_q.weight, to_k.weight, to_v.weight,
               to_out.weight, norm_q.weight, norm_k.weight,
               layer.post_attention_layernorm_moe_gen.weight, mlp.gate_proj.weight,
               mlp.up_proj.weight, mlp.down_proj.weight)
    with span(f"layer {layer_index} forward"):
        y = _Layer.apply(x.contiguous(), cos.contiguous(), sin.contiguous(), layer, schedule,
                         text_k, text_v, valid, max(0, len(text.keys) - layer_index - 1), *weights)
    if len(sizes) == 1:
        return [y]
    pieces = list(y.split(sizes, dim=1))
    y._agb_sizes = tuple(sizes)
    for index, piece in enumerate(pieces):   # the next layer recognises them and takes y itself
        piece._agb_whole, piece._agb_index = y, index
    return pieces
