"""Linear layers on the tcgen05 GEMM.

``linear(x, W, b)`` computes ``x @ W.T + b``.  For bf16 CUDA tensors the forward GEMM, the
input gradient (``dY @ W``) and the weight gradient (``dY.T @ x``) all run on the same
TMA-fed, TMEM-accumulating kernel with the operand majorness selected per call, so no
operand is ever transposed in memory.  Results are row-invariant: a row of the output
depends only on that row of ``x`` (fixed tile shapes and K order), which the block-causal
replay contract relies on.

Parity: every ``nn.Linear`` of the reference (``wm/networks/cosmos3/layers.py:83-97,173-200``),
which run on cuBLAS there.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native

__all__ = ["adjoin", "gemm", "joined", "joint_linear", "linear", "linear_residual", "rows_linear"]


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = True,
         out: torch.Tensor | None = None, accumulate: bool = False,
         bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``op(a) @ op(b)`` for 2-D bf16 CUDA tensors on the tcgen05 kernel.

    ``trans_b=True`` (default) treats ``b`` as ``[N, K]`` (the ``nn.Linear`` weight layout);
    ``trans_a=True`` treats ``a`` as ``[K, M]``.  ``accumulate`` adds into ``out``.
    """
    C = native.ext()
    native.count()
    return C.gemm(a, b, bool(trans_a), bool(trans_b), out, bool(accumulate), bias, residual,
                  out_dtype or a.dtype)


def _gemm_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    n, k = weight.shape
    return (weight.dtype == x.dtype and weight.is_contiguous() and k % 8 == 0 and n % 8 == 0
            and x.numel() > 0)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, weight)
        ctx.save_for_forward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        out = gemm(x2, weight, bias=bias)
        return out.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def jvp(ctx, x_tangent, weight_tangent, bias_tangent):
        """Forward mode: ``d(x W^T + b) = dx W^T + x dW^T + db`` on the same tensor-core kernel
        (the exact R1/R2 penalties push a direction through the frozen backbone this way)."""
        x2, weight = ctx.saved_tensors
        tangent = None
        if x_tangent is not None:
            rows = x_tangent.reshape(-1, x_tangent.shape[-1]).to(x2.dtype)
            tangent = gemm(rows if rows.is_contiguous() else rows.contiguous(), weight)
        if weight_tangent is not None:
            moved = weight_tangent.to(weight.dtype).contiguous()
            tangent = gemm(x2, moved) if tangent is None else gemm(x2, moved, out=tangent, accumulate=True)
        if tangent is None:
            tangent = x2.new_zeros(x2.shape[0], weight.shape[0])
        if bias_tangent is not None:
            tangent = tangent + bias_tangent.to(tangent.dtype)
        return tangent.view(*ctx.shape[:-1], weight.shape[0])

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        x2, weight = ctx.saved_tensors
        g2 = grad.reshape(-1, grad.shape[-1])
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(g2, weight, trans_b=False).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            dw = gemm(g2, x2, trans_a=True, trans_b=False)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = g2.float().sum(0).to(grad.dtype)
        return dx, dw, db


class _RowsLinear(torch.autograd.Function):
    """A few FP32 rows through a wide linear layer, evaluated in FP32 with the weights read in their
    own type (``csrc/rows_linear.cu``); gradients in FP32, cast to the parameters' type."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        native.count()
        ctx.save_for_backward(x, weight)
        ctx.bias_dtype = None if bias is None else bias.dtype
        return native.ext().rows_linear_fwd(x, weight, bias)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        x, weight = ctx.saved_tensors
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        native.count(2)
        dx, dw, db = native.ext().rows_linear_bwd(grad.contiguous(), x, weight, need_dx, need_dw)
        return (dx, dw.to(weight.dtype) if ctx.needs_input_grad[1] else None,
                db.to(ctx.bias_dtype) if ctx.needs_input_grad[2] and ctx.bias_dtype is not None else None)


def rows_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T + bias`` in FP32 for a few FP32 rows ``x`` (the timestep embedder): on CUDA a
    kernel that reads bf16 or fp32 weights in place, elsewhere PyTorch with upcast weights.

    Parity: the FP32 MLP of ``wm/networks/cosmos3/layers.py:100-128`` (cuBLAS ``sgemm`` there)."""
    import torch.autograd.forward_ad as fwAD

    ok = (x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.shape[0] <= 256 and x.shape[1] % 8 == 0
          and weight.dtype in (torch.bfloat16, torch.float32) and weight.dim() == 2
          and (bias is None or bias.dtype == weight.dtype) and native.available()
          and fwAD.unpack_dual(x).tangent is None and fwAD.unpack_dual(weight).tangent is None)
    if ok:
        return _RowsLinear.apply(x.contiguous(), weight.contiguous(), None if bias is None else bias.contiguous())
    return F.linear(x, weight.float(), None if bias is None else bias.float())


def linear_residual(x: torch.Tensor, module, residual: torch.Tensor) -> torch.Tensor:
    """``residual + module(x)`` for a bias-free linear ``module``.  Where no gradient or tangent is
    wanted on the CUDA bf16 path the sum happens in the GEMM's epilogue (FP32 accumulator plus
    residual, rounded once, as the whole-layer training path does); otherwise it is the plain sum."""
    import torch.autograd.forward_ad as fwAD

    weight = module.weight
    fused = (type(module).__name__ == "Linear" and module.bias is None and native.use(x) and _gemm_ok(x, weight)
             and x.shape[-1] % 8 == 0 and residual.dtype == x.dtype and residual.shape[:-1] == x.shape[:-1]
             and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad or residual.requires_grad))
             and fwAD.unpack_dual(x).tangent is None and fwAD.unpack_dual(residual).tangent is None)
    if not fused:
        return residual + module(x)
    native.count()
    rows = x.reshape(-1, x.shape[-1])
    res = residual.reshape(-1, residual.shape[-1])
    out = native.ext().gemm(rows if rows.is_contiguous() else rows.contiguous(), weight, False, True, None, False,
                            None, res if res.is_contiguous() else res.contiguous(), torch.bfloat16)
    return out.view(*x.shape[:-1], weight.shape[0])


def joined(parts):
    """One ``[sum of rows, K]`` view over matrices that lie back to back in one storage, in
    this order (the optimizer engine's flat parameter buffer and ``prepare_serving`` lay q|k|v and
    gate|up out that way); None when they do not."""
    first = parts[0]
    if any(p is None for p in parts):
        return None
    at, storage = first.data_ptr(), first.untyped_storage().data_ptr()
    for p in parts:
        if (p.dim() != 2 or not p.is_contiguous() or p.shape[1] != first.shape[1] or p.dtype != first.dtype
                or p.data_ptr() != at or p.untyped_storage().data_ptr() != storage):
            return None
        at += p.numel() * p.element_size()
    rows = sum(p.shape[0] for p in parts)
    return first.detach().as_strided((rows, first.shape[1]), (first.shape[1], 1))


def adjoin(parameters) -> None:
    """Move the data of 2-D parameters of equal width into one buffer, back to back, so that
    :func:`joined` finds them (a one-time copy; the old storages are released)."""
    parameters = list(parameters)
    if joined([p.data for p in parameters]) is not None:
        return
    width = parameters[0].shape[1]
    assert all(p.dim() == 2 and p.shape[1] == width and p.dtype == parameters[0].dtype for p in parameters)
    buffer = torch.empty(sum(p.shape[0] for p in parameters), width, dtype=parameters[0].dtype,
                         device=parameters[0].device)
    at = 0
    for p in parameters:
        view = buffer[at:at + p.shape[0]]
        view.copy_(p.data)
        p.data = view
        at += p.shape[0]


def joint_linear(x: torch.Tensor, modules) -> torch.Tensor | None:
    """``x`` through several bias-free linears as ONE GEMM over their adjacent weights:
    ``[..., sum of out features]``, or None when that does not apply (weights not adjacent, a
    bias, gradients or tangents wanted, not the CUDA bf16 path).  An output column is the same
    K-ordered sum as from one GEMM per weight."""
    weights = [m.weight for m in modules]
    if any(m.bias is not None for m in modules) or not native.use(x) or x.shape[-1] % 8:
        return None
    if torch.is_grad_enabled() and (x.requires_grad or any(w.requires_grad for w in weights)):
        return None
    # plain linears only: a subclass with its own forward (LoRA) must not be bypassed
    if any(type(m).__name__ != "Linear" for m in modules) or not _gemm_ok(x, weights[0]):
        return None
    import torch.autograd.forward_ad as fwAD

    if fwAD.unpack_dual(x).tangent is not None:
        return None
    weight = joined(weights)
    if weight is None:
        return None
    return _Linear.apply(x, weight, None)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    if native.use(x) and _gemm_ok(x, weight) and x.shape[-1] % 8 == 0:
        return _Linear.apply(x, weight, bias)  # reverse mode and forward mode (dual inputs) alike
    return F.linear(x, weight, bias)
