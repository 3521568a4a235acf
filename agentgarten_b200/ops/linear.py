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

__all__ = ["gemm", "linear"]


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


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    if native.use(x) and _gemm_ok(x, weight) and x.shape[-1] % 8 == 0:
        return _Linear.apply(x, weight, bias)  # reverse mode and forward mode (dual inputs) alike
    return F.linear(x, weight, bias)
