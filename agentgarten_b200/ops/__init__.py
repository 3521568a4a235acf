"""Operator facade.

Every operator has two implementations that compute the same function:

* the sm_100a CUDA kernels of ``agentgarten_b200/csrc`` (loaded through
  :mod:`agentgarten_b200.ops.native`), used for bf16 tensors on a CUDA device, and
* the PyTorch definitions in :mod:`agentgarten_b200.ops.reference`, used on CPU and for
  other dtypes, and as the numerical oracle in the tests.

On a CUDA device a missing extension is an error, never a silent fallback.
"""

from __future__ import annotations

import torch
import torch.autograd.forward_ad as fwAD

from . import native, reference
from .attention import attention, attention_jvp, planned_attention
from .linear import adjoin, joined, joint_linear, linear, linear_residual, rows_linear
from .pointwise import (
    gated_residual,
    head_norm_rope,
    norm_modulate,
    rf_interpolate,
    rf_x0,
    dmd_target,
    rms_norm,
    rms_norm_add,
    rotary,
    silu_mul,
    silu_mul_pair,
)

__all__ = [
    "adjoin",
    "attention",
    "attention_jvp",
    "gated_residual",
    "head_norm_rope",
    "joined",
    "joint_linear",
    "linear",
    "linear_residual",
    "native",
    "norm_modulate",
    "planned_attention",
    "reference",
    "rf_interpolate",
    "rf_x0",
    "dmd_target",
    "rms_norm",
    "rows_linear",
    "rms_norm_add",
    "rotary",
    "silu_mul",
    "silu_mul_pair",
]
