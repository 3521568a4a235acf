"""Stand-in for Transformer Engine, which is absent from the offline image.

The reference optimizer needs exactly two things from it: ``multi_tensor_applier`` and the
multi-tensor Adam entry points of ``transformer_engine_torch``.  Both are provided on
PyTorch's own fused multi-tensor AdamW kernel (``torch._fused_adamw_``), the closest library
equivalent of Transformer Engine's kernel.
"""

__version__ = "0.0-standin"
