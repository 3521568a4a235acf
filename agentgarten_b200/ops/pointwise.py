"""Row-wise and element-wise operators with hand-written forward/backward kernels.

Parity: the fused serving kernels of the reference (``wm/kernels/gen_layer.py:29-119``:
RMSNorm with optional residual add, per-head RMSNorm + rotary, SiLU·mul) and the
rectified-flow pointwise steps (``wm/models/flow.py:49-59``).
"""

from __future__ import annotations

import torch

from . import native, reference

__all__ = ["head_norm_rope", "rf_interpolate", "rf_x0", "rms_norm", "rms_norm_add", "rotary",
           "silu_mul"]


def _plain(*tensors: torch.Tensor) -> bool:
    """Kernels handle the ordinary reverse-mode/no-grad case; exotic autograd modes
    (forward-mode duals, double backward) go through the PyTorch definitions."""
    import torch.autograd.forward_ad as fwAD

    return not any(fwAD.unpack_dual(t).tangent is not None for t in tensors)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        C = native.ext()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        out, rstd = C.rms_norm_fwd(x2, weight.contiguous(), float(eps))
        native.count()
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return out.view(x.shape)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        C = native.ext()
        x2, weight, rstd = ctx.saved_tensors
        g2 = grad.reshape(-1, grad.shape[-1]).contiguous()
        dx, dw = C.rms_norm_bwd(g2, x2, weight.contiguous(), rstd)
        native.count(2)
        return dx.view(ctx.shape), dw.to(weight.dtype), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if native.use(x) and weight.dtype == x.dtype and _plain(x, weight) and x.shape[-1] % 8 == 0:
        return _RMSNorm.apply(x, weight, eps)
    return reference.rms_norm(x, weight, eps)


def rms_norm_add(x, addend, weight, eps):
    if native.use(x) and not torch.is_grad_enabled() and weight.dtype == x.dtype:
        C = native.ext()
        shape = x.shape
        total, out = C.rms_norm_add_fwd(
            x.reshape(-1, shape[-1]).contiguous(), addend.reshape(-1, shape[-1]).contiguous(),
            weight.contiguous(), float(eps))
        native.count()
        return total.view(shape), out.view(shape)
    total = x + addend
    return total, rms_norm(total, weight, eps)


def _column_block(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor | None:
    """``t`` as a 2-D ``[rows, H]`` view with unit inner stride (a chunk of a wider projection), or None."""
    if t.shape != like.shape or t.dtype != like.dtype or t.stride(-1) != 1:
        return None
    try:
        flat = t.view(-1, t.shape[-1])
    except RuntimeError:
        return None
    return flat if flat.stride(0) % 8 == 0 and flat.data_ptr() % 16 == 0 else None


def norm_modulate(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor,
                  eps: float) -> torch.Tensor:
    """AdaLN input: ``rms_norm(x) * (1 + scale) + shift`` in one pass when no gradient is wanted
    (``wm/networks/cosmos3/layers.py:269-276`` with the ``adaln`` option)."""
    if native.use(x) and weight.dtype == x.dtype and x.shape[-1] % 8 == 0 and not (
            torch.is_grad_enabled() and any(t.requires_grad for t in (x, weight, scale, shift))):
        rows = x.reshape(-1, x.shape[-1])
        sc, sh = _column_block(scale, x), _column_block(shift, x)
        if rows.is_contiguous() and sc is not None and sh is not None and sc.stride(0) == sh.stride(0):
            native.count()
            return native.ext().norm_modulate(rows, weight.contiguous(), sc, sh, float(eps)).view(x.shape)
    return rms_norm(x, weight, eps) * (1 + scale) + shift


def gated_residual(hidden: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """AdaLN output: ``hidden + gate * y`` in one pass when no gradient is wanted."""
    if native.use(hidden) and y.dtype == hidden.dtype and y.shape == hidden.shape and hidden.shape[-1] % 8 == 0 \
            and not (torch.is_grad_enabled() and any(t.requires_grad for t in (hidden, gate, y))):
        g = _column_block(gate, hidden)
        if g is not None and hidden.is_contiguous() and y.is_contiguous():
            native.count()
            width = hidden.shape[-1]
            return native.ext().gated_residual(hidden.view(-1, width), g, y.view(-1, width)).view(hidden.shape)
    return hidden + gate * y


def rotary(value, cos, sin):
    return reference.rotary(value, cos, sin)


class _HeadNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, value, weight, cos, sin, eps):
        C = native.ext()
        value = value.contiguous()
        out, rstd = C.head_norm_rope_fwd(value, weight.contiguous(), cos.contiguous(),
                                         sin.contiguous(), float(eps))
        native.count()
        ctx.save_for_backward(value, weight, cos, sin, rstd)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        C = native.ext()
        value, weight, cos, sin, rstd = ctx.saved_tensors
        dx, dw = C.head_norm_rope_bwd(grad.contiguous(), value, weight.contiguous(),
                                      cos.contiguous(), sin.contiguous(), rstd, None)
        native.count(2)
        return dx, dw.to(weight.dtype), None, None, None


def _row_strided(value) -> bool:
    """``[B, N, H, 128]`` dense over (H, 128) with rows at a constant stride: a column slice of a
    wider matrix, which the kernel reads in place."""
    return (value.dim() == 4 and value.stride(3) == 1 and value.stride(2) == 128 and value.stride(1) % 8 == 0
            and (value.shape[0] == 1 or value.stride(0) == value.shape[1] * value.stride(1)))


def head_norm_rope(value, weight, cos, sin, eps):
    """Per-head RMSNorm over ``D`` then rotate-half RoPE; ``value`` is ``[B, N, H, D]``."""
    if (native.use(value) and value.shape[-1] == 128 and weight.dtype == value.dtype
            and cos.dtype == value.dtype and _plain(value, weight)):
        if not (torch.is_grad_enabled() and (value.requires_grad or weight.requires_grad)) and _row_strided(value):
            native.count()
            return native.ext().head_norm_rope_fwd(value, weight.contiguous(), cos.contiguous(),
                                                   sin.contiguous(), float(eps))[0]
        return _HeadNormRope.apply(value, weight, cos, sin, eps)
    return reference.head_norm_rope(value, weight, cos, sin, eps)


class _SiluMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        C = native.ext()
        gate, up = gate.contiguous(), up.contiguous()
        ctx.save_for_backward(gate, up)
        native.count()
        return C.silu_mul_fwd(gate, up)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        C = native.ext()
        gate, up = ctx.saved_tensors
        native.count()
        dgate, dup = C.silu_mul_bwd(grad.contiguous(), gate, up)
        return dgate, dup


def silu_mul(gate, up):
    if native.use(gate) and _plain(gate, up) and gate.numel() % 8 == 0:
        return _SiluMul.apply(gate, up)
    return reference.silu_mul(gate, up)


def silu_mul_pair(both):
    """``silu(gate) * up`` for ``both = [gate | up]`` along the last dimension (the product of a
    joint gate|up GEMM); no gradient."""
    width = both.shape[-1] // 2
    if native.use(both) and both.is_contiguous() and width % 8 == 0 and not both.requires_grad:
        native.count()
        return native.ext().silu_mul_pair(both.view(-1, 2 * width)).view(*both.shape[:-1], width)
    return reference.silu_mul(both[..., :width], both[..., width:])


def rf_interpolate(x0, noise, sigma):
    """``(1 - sigma) * x0 + sigma * noise`` with ``sigma`` ``[B]`` or ``[B, T]``."""
    if (native.use(x0, dtypes=(torch.float32, torch.bfloat16)) and x0.ndim == 5
            and not torch.is_grad_enabled() and x0.dtype == noise.dtype and _plain(x0, noise)):
        C = native.ext()
        native.count()
        return C.rf_combine(x0.contiguous(), noise.contiguous(), sigma.float().contiguous(), 0)
    return reference.rf_interpolate(x0, noise, sigma)


def rf_x0(noisy, sigma, velocity):
    """``noisy - sigma * velocity``."""
    if (native.use(noisy, dtypes=(torch.float32, torch.bfloat16)) and noisy.ndim == 5
            and not torch.is_grad_enabled() and noisy.dtype == velocity.dtype
            and _plain(noisy, velocity)):
        C = native.ext()
        native.count()
        return C.rf_combine(noisy.contiguous(), velocity.contiguous(),
                            sigma.float().contiguous(), 1)
    return reference.rf_x0(noisy, sigma, velocity)


def dmd_target(estimate, by_fake, by_teacher):
    """Distribution-matching target in FP64 and the root mean square of its step.

    Per sample ``spread = max(mean |estimate - by_teacher|, 1e-5)``; the step is
    ``(by_fake - by_teacher) / spread`` and the target ``estimate - step`` (reference
    ``wm/models/dmd.py:496-507``).  On a GPU two launches replace the chain of FP64 tensor
    expressions; the sums run in a fixed order.
    """
    if (native.use(estimate, dtypes=(torch.float32,)) and not torch.is_grad_enabled()
            and by_fake.dtype == by_teacher.dtype == torch.float32 and estimate.ndim >= 2
            and estimate.shape == by_fake.shape == by_teacher.shape and estimate.shape[0] <= 65535):
        C = native.ext()
        native.count(2)
        target, squares = C.dmd_target(estimate.contiguous(), by_fake.contiguous(), by_teacher.contiguous())
        return target, (squares.sum() / max(1, estimate.numel())).sqrt().float()
    wide, teacher = estimate.double(), by_teacher.double()
    spread = (wide - teacher).abs().flatten(1).mean(1).clamp_min(1e-5)
    step = (by_fake.double() - teacher) / spread.view(-1, *([1] * (estimate.ndim - 1)))
    return wide - step, step.float().square().mean().sqrt()
