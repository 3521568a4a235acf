"""Stride-1 convolutions of channels-last bf16 / fp16 activations on the tensor cores.

The codecs spend their time in 3x3x3 causal convolutions and 3x3 frame convolutions
(``wm/codecs/wan22.py:29-55`` ``CausalConv3d``, ``wm/codecs/wan22.py:97-160`` ``Resample``,
``ResidualBlock``).  On a CUDA device they run as one implicit-GEMM kernel
(``csrc/conv3d.cu``): TMA loads the input patch shifted by each kernel tap directly from
the channels-last volume (out-of-frame positions read as zero: the spatial padding), the
products accumulate in TMEM, and bias, the residual branch and a ReLU are applied in the
epilogue.  The TAEHV decoders (``wm/codecs/_taehv/taehv.py:30-75`` ``MemBlock``) use the same
kernel in fp16.
Everything else — other strides, dtypes, devices, or inputs that need gradients — goes to
``torch.nn.functional``.
"""

from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from . import native

__all__ = ["conv_frames", "conv_volume", "conv_volume_causal", "depthwise_frames", "eligible", "packed_weight"]


def _weight_key(weight: torch.Tensor, dtype: torch.dtype) -> tuple:
    """Identity of a weight's current value (inference tensors carry no version counter)."""
    version = -1 if weight.is_inference() else weight._version
    return (version, weight.data_ptr(), weight.device, dtype)


def packed_weight(conv: torch.nn.Module, dtype: torch.dtype = torch.bfloat16
                  ) -> tuple[torch.Tensor, torch.Tensor | None]:
    """``[Cout', taps, Cin]`` copy of a convolution's weight and its bias in ``dtype``, cached on
    the module.  ``Cout'`` is ``Cout`` rounded up to a multiple of 8 (zero rows)."""
    weight = conv.weight
    key = _weight_key(weight, dtype)
    cached = getattr(conv, "_packed_for_kernel", None)
    if cached is None or cached[0] != key:
        w = weight.detach()
        if w.ndim == 4:
            w = w.unsqueeze(2)
        packed = w.permute(0, 2, 3, 4, 1).reshape(w.shape[0], -1, w.shape[1])
        packed = packed.to(dtype).contiguous()
        bias = None if conv.bias is None else conv.bias.detach().to(dtype).contiguous()
        pad = -packed.shape[0] % 8
        if pad:
            packed = torch.cat((packed, packed.new_zeros(pad, *packed.shape[1:])))
            bias = None if bias is None else torch.cat((bias, bias.new_zeros(pad)))
        cached = (key, packed, bias)
        conv._packed_for_kernel = cached
    return cached[1], cached[2]


def eligible(conv: torch.nn.Module, x: torch.Tensor) -> bool:
    """Whether ``conv(x)`` can run in the kernel: bf16 or fp16 on CUDA, stride 1, 'same' in
    space, unpadded in time, input channels a multiple of 8, no gradient wanted."""
    if not native.use(x, dtypes=(torch.bfloat16, torch.float16)):  # raises when the extension is missing
        return False
    if os.environ.get("AGB200_LIBRARY_CONV") == "1":  # measure against cuDNN
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
    return conv.in_channels % 8 == 0 and x.shape[1] == conv.in_channels and conv.weight.dtype == x.dtype


def _rows(x: torch.Tensor) -> torch.Tensor:
    """Channels-last rows ``[..., C]`` of a channel-first tensor (a view when it already is)."""
    order = (0, *range(2, x.ndim), 1)
    rows = x.permute(order)
    return rows if rows.is_contiguous() else rows.contiguous()


def _finish(out: torch.Tensor, residual: torch.Tensor | None, relu: bool) -> torch.Tensor:
    if residual is not None:
        out = out + residual
    return F.relu(out) if relu else out


def _launch(conv, rows: torch.Tensor, residual: torch.Tensor | None, kernel: tuple, relu: bool,
            history: torch.Tensor | None = None, causal: bool = False) -> torch.Tensor:
    """The kernel on channels-last rows ``[B, T, H, W, Cin]`` -> ``[B, T', H, W, Cout]``."""
    weight, bias = packed_weight(conv, rows.dtype)
    padded = weight.shape[0] != conv.out_channels
    native.count()
    if padded and (residual is not None or relu):
        out = native.ext().conv3d(rows, weight, bias, None, *kernel, False, history, causal)
        return _finish(out[..., : conv.out_channels], residual, relu)
    out = native.ext().conv3d(rows, weight, bias, residual, *kernel, relu, history, causal)
    return out[..., : conv.out_channels] if padded else out


def conv_volume(conv: torch.nn.Conv3d, x: torch.Tensor, residual: torch.Tensor | None = None,
                relu: bool = False) -> torch.Tensor:
    """``act(conv(x) (+ residual))`` for ``x`` ``[B, C, T, H, W]``; time is not padded."""
    if not eligible(conv, x) or x.shape[2] < conv.kernel_size[0]:
        out = F.conv3d(x, conv.weight, conv.bias, conv.stride, conv.padding, conv.dilation, conv.groups)
        return _finish(out, residual, relu)
    out = _launch(conv, _rows(x), None if residual is None else _rows(residual), conv.kernel_size, relu)
    return out.permute(0, 4, 1, 2, 3)


def conv_volume_causal(conv: torch.nn.Conv3d, x: torch.Tensor, history: torch.Tensor | None,
                       residual: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
    """Causal form for ``eligible`` calls: the ``kt - 1`` frames before ``x`` are the last frames
    of ``history`` (``[B, C, <= kt - 1, H, W]`` or ``None``) preceded by zeros; the kernel reads
    them where they are, nothing is joined.  Returns as many frames as ``x`` has."""
    past = None
    if history is not None and history.shape[2] > 0:
        past = _rows(history[:, :, -(conv.kernel_size[0] - 1):])
    out = _launch(conv, _rows(x), None if residual is None else _rows(residual), conv.kernel_size, relu,
                  history=past, causal=True)
    return out.permute(0, 4, 1, 2, 3)


def conv_frames(conv: torch.nn.Conv2d, x: torch.Tensor, residual: torch.Tensor | None = None,
                relu: bool = False) -> torch.Tensor:
    """``act(conv(x) (+ residual))`` for frames ``x`` ``[N, C, H, W]``."""
    if not eligible(conv, x):
        out = F.conv2d(x, conv.weight, conv.bias, conv.stride, conv.padding, conv.dilation, conv.groups)
        return _finish(out, residual, relu)
    res = None if residual is None else _rows(residual).unsqueeze(0)
    out = _launch(conv, _rows(x).unsqueeze(0), res, (1, *conv.kernel_size), relu)
    return out.squeeze(0).permute(0, 3, 1, 2)


def depthwise_frames(conv: torch.nn.Conv2d, x: torch.Tensor) -> torch.Tensor:
    """Depthwise ``conv(x)`` for frames ``[N, C, H, W]`` (``groups == C``, square odd kernel up
    to 7, stride 1, 'same' padding) in the register-tiled kernel of ``csrc/depthwise.cu``; the
    7x7 stage of the wide TAEHV decoder blocks (``wm/codecs/_taehv/taehv.py:52-75``)."""
    k = conv.kernel_size[0]
    fits = (native.use(x, dtypes=(torch.bfloat16, torch.float16))
            and os.environ.get("AGB200_LIBRARY_CONV") != "1"
            and conv.weight.dtype == x.dtype
            and not (torch.is_grad_enabled() and (x.requires_grad or conv.weight.requires_grad))
            and conv.groups == conv.in_channels == conv.out_channels == x.shape[1]
            and conv.kernel_size == (k, k) and k in (3, 5, 7) and tuple(conv.padding) == (k // 2, k // 2)
            and tuple(conv.stride) == (1, 1) and tuple(conv.dilation) == (1, 1)
            and conv.padding_mode == "zeros" and x.shape[1] % 8 == 0)
    if not fits:
        return F.conv2d(x, conv.weight, conv.bias, conv.stride, conv.padding, conv.dilation, conv.groups)
    weight = conv.weight
    key = _weight_key(weight, x.dtype)
    cached = getattr(conv, "_packed_for_kernel", None)
    if cached is None or cached[0] != key:
        taps = weight.detach().reshape(weight.shape[0], k * k).t().contiguous()  # [k*k, C]
        bias = None if conv.bias is None else conv.bias.detach().contiguous()
        cached = (key, taps, bias)
        conv._packed_for_kernel = cached
    native.count()
    out = native.ext().depthwise(_rows(x), cached[1], cached[2], k)
    return out.permute(0, 3, 1, 2)
