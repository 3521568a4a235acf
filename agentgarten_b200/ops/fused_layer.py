"""Whole-layer execution of a generation layer on the CUDA kernels.

Placeholder gate: the op-by-op path in ``networks/cosmos3/layers.py`` is used until the
fused layer (manual forward/backward over concatenated chunks, attention outputs kept,
everything else recomputed) is enabled for a configuration.
"""

from __future__ import annotations


def eligible(layer, chunks) -> bool:
    return False


def run(layer, chunks, ropes, attention, layer_index):
    raise NotImplementedError
