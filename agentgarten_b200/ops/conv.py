"""Stride-1 convolutions of channels-last bf16 activations on the tensor cores.

The codecs spend their time in 3x3x3 causal convolutions and 3x3 frame convolutions
(``wm/codecs/wan22.py:29-55`` ``CausalConv3d``, ``wm/codecs/wan22.py:97-160`` ``Resample``,
``ResidualBlock``).  On a CUDA device they run as one implicit-GEMM kernel
(``csrc/conv3d.cu``): TMA loads the input patch shifted by each kernel tap directly from
the channels-last volume (out-of-frame positions read as zero: the spatial padding), the
products accumulate in TMEM, and bias plus the residual branch are added in the epilogue.
Everything else — other strides, dtypes, devices, or inputs that need gradients — goes to
``torch.nn.functional``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native

__all__ = ["conv_frames", "conv_volume", "eligible", "packed_weight"]


def packed_weight(conv: torch.nn.Module) -> tuple[torch.Tensor, torch.Tensor | None]:
    """``[Cout, taps, Cin]`` bf16 copy of a convolution's weight and its bf16 bias, cached on the module."""
    weight = conv.weight
    key = (weight._version, weight.data_ptr(), weight.device)
    cached = getattr(conv, "_packed_for_kernel", None)
    if cached is None or cached[0] != key:
        w = weight.detach()
        if w.ndim == 4:
            w = w.unsqueeze(2)
        packed = w.permute(0, 2, 3, 4, 1).reshape(w.shape[0], -1, w.shape[1])
        packed = packed.to(torch.bfloat16).contiguous()
        bias = None if conv.bias is None else conv.bias.detach().to(torch.bfloat16).contiguous()
        cached = (key, packed, bias)
        conv._packed_for_kernel = cached
    return cached[1], cached[2]


def eligible(conv: torch.nn.Module, x: torch.Tensor) -> bool:
    """Whether ``conv(x)`` can run in the kernel: bf16 on CUDA, stride 1, 'same' in space,
    unpadded in time, channel counts multiples of 8, no gradient wanted."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and native.available()):
        return False
    if torch.is_grad_enabled() and (x.requires_grad or conv.weight.requires_grad):
        return False
    spatial = len(conv.kernel_size)
    if any(s != 1 for s in conv.stride) or any(d != 1 for d in conv.dilation) or conv.groups != 1:
        return False
    if conv.padding_mode != "zeros" or isinstance(conv.padding, str):
        return False
    kernel, padding = tuple(conv.kernel_size), tuple(conv.padding)
    if spatial == 3 and padding[0] != 0:
        return False
    if any(k % 2 == 0 or p != k // 2 for k, p in zip(kernel[-2:], padding[-2:])):
        return False
    return conv.in_channels % 8 == 0 and conv.out_channels % 8 == 0 and x.shape[1] == conv.in_channels


def _rows(x: torch.Tensor) -> torch.Tensor:
    """Channels-last rows ``[..., C]`` of a channel-first tensor (a view when it already is)."""
    order = (0, *range(2, x.ndim), 1)
    rows = x.permute(order)
    return rows if rows.is_contiguous() else rows.contiguous()


def conv_volume(conv: torch.nn.Conv3d, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``conv(x) (+ residual)`` for ``x`` ``[B, C, T, H, W]``; time is not padded."""
    if not eligible(conv, x) or x.shape[2] < conv.kernel_size[0]:
        out = F.conv3d(x, conv.weight, conv.bias, conv.stride, conv.padding, conv.dilation, conv.groups)
        return out if residual is None else out + residual
    weight, bias = packed_weight(conv)
    native.count()
    out = native.ext().conv3d(_rows(x), weight, bias, None if residual is None else _rows(residual),
                              *conv.kernel_size)
    return out.permute(0, 4, 1, 2, 3)


def conv_frames(conv: torch.nn.Conv2d, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``conv(x) (+ residual)`` for frames ``x`` ``[N, C, H, W]``."""
    if not eligible(conv, x):
        out = F.conv2d(x, conv.weight, conv.bias, conv.stride, conv.padding, conv.dilation, conv.groups)
        return out if residual is None else out + residual
    weight, bias = packed_weight(conv)
    native.count()
    res = None if residual is None else _rows(residual).unsqueeze(0)
    out = native.ext().conv3d(_rows(x).unsqueeze(0), weight, bias, res, 1, *conv.kernel_size)
    return out.squeeze(0).permute(0, 3, 1, 2)
