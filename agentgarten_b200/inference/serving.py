"""Serving preparation of a generation tower.

``prepare_serving`` switches the network to its inference configuration: parameters frozen
and in eval mode, every layer routed through the CUDA kernels (they are the default
operator path for bf16 CUDA tensors) and — with ``cuda_graphs=True`` — whole-step CUDA
graph replay enabled for streams created from the network afterwards.  A stream captures
one graph per (cache fill level, denoise|commit); in steady state a denoise call is a single
graph launch covering all layers, the cache writes, attention and the output projection.
``release_serving`` drops the option (streams created later run eagerly).

Parity: reference ``wm/inference/serving.py:17-96`` (per-layer graphs around Triton
``project``/``finish`` with attention left outside the graphs).
"""

from __future__ import annotations

import torch

__all__ = ["prepare_serving", "release_serving"]


def prepare_serving(network: torch.nn.Module, *, dynamic: bool = False, cuda_graphs: bool = True,
                    inductor: bool = False, tensor_parallel: object = None,
                    max_tokens: int = 8192) -> torch.nn.Module:
    """``dynamic`` and ``inductor`` are accepted for call compatibility: shapes are handled by
    per-shape graphs and nothing is traced or compiled here.

    ``tensor_parallel``: ``True`` (all ranks of the default process group) or a process group
    shards heads and MLP columns over those GPUs of one node; streams then run the fused
    GEMM + peer-memory kernels of :mod:`agentgarten_b200.parallel.tensor_parallel`.  Every
    rank must hold the full weights when this is called and must drive its stream with the
    same inputs in the same order.  ``max_tokens`` bounds the tokens of one chunk.
    """
    del dynamic, inductor
    network.eval()
    network.requires_grad_(False)
    on_cuda = next(network.parameters()).is_cuda
    network._serving_options = {"cuda_graphs": bool(cuda_graphs) and on_cuda}
    network._tensor_parallel = None
    if on_cuda:
        _adjoin_projections(network)
    if tensor_parallel is not None and tensor_parallel is not False:
        if not on_cuda:
            raise ValueError("tensor-parallel serving needs CUDA devices")
        from agentgarten_b200.parallel.tensor_parallel import TensorParallelServing

        group = None if tensor_parallel is True else tensor_parallel
        network._tensor_parallel = TensorParallelServing(network, group, max_tokens=max_tokens)
    return network


def _adjoin_projections(network: torch.nn.Module) -> None:
    """Lay the q | k | v and the gate | up weights of every layer out back to back (a one-time
    copy, one layer at a time), so that a served step runs each group as one GEMM: at the 3120
    rows of a streamed block the k and v projections alone fill less than a wave of SMs."""
    from agentgarten_b200 import ops

    for module in network.modules():
        groups = []
        if callable(getattr(module, "parts", None)):
            groups.append(module.parts()[:3])
        if all(hasattr(module, name) for name in ("gate_proj", "up_proj", "down_proj")):
            groups.append((module.gate_proj, module.up_proj))
        for group in groups:
            if all(isinstance(m, torch.nn.Linear) and m.bias is None and m.weight.dim() == 2 for m in group) \
                    and len({m.weight.shape[1] for m in group}) == 1:
                ops.adjoin([m.weight for m in group])


def release_serving(network: torch.nn.Module) -> torch.nn.Module:
    network._serving_options = None
    network._tensor_parallel = None
    return network
