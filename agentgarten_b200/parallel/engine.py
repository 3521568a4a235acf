"""Placement of a network on the job's GPUs.

``parallelize_network`` casts a network to its parameter dtype, materialises meta
parameters on the device, enables context parallelism, installs activation recomputation
and records the data-parallel group the network's gradients are reduced over.

Data parallelism is *sharded-optimizer replication*: on a B200 (180 GB) the bf16
parameters of a 7 B tower are kept whole on every GPU, so no parameter all-gather sits in
front of every layer; gradients are reduce-scattered once per update, each rank runs Adam
on its shard of the FP32 master/moment state, and the updated bf16 shards are written
straight into every peer's parameter buffer.  The three steps are one peer-memory kernel
pair (see :mod:`agentgarten_b200.parallel.zero`).  Shard ownership follows the
"chunk dim 0 per parameter" rule of FSDP2, so sharded checkpoints are interchangeable.

Parity: reference ``wm/infra/parallel.py:58-254`` (``ParallelConfig``, meshes, activation
checkpointing, FSDP2 wrapping, meta materialisation).
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field
from enum import StrEnum
from math import prod
from typing import Any

import torch
import torch.distributed as dist
from torch import nn
from torch.utils.checkpoint import checkpoint

from agentgarten_b200.infra.distributed import get_local_world_size

from .network import ParallelNetwork

__all__ = [
    "replicated_parameter_bytes",
    "ATTENTION_SAVE_OPS",
    "ActivationCheckpointing",
    "ParallelConfig",
    "ParallelNetwork",
    "init_meshes",
    "parallelize_network",
]

# Names of the operators whose outputs are kept under selective recomputation.
ATTENTION_SAVE_OPS = (r"scaled_dot_product", r"flash_attn", r"fmha")


class ActivationCheckpointing(StrEnum):
    NONE = "none"
    SELECTIVE = "selective"
    FULL = "full"


@dataclass(frozen=True)
class ParallelConfig:
    parameter_dtype: str = "bfloat16"
    fully_shard: bool = True
    # None: one shard group over all ranks of a node; (nodes, local) on several nodes.
    fsdp_mesh_shape: tuple[int, ...] | None = None
    context_parallel_size: int = 1
    activation_checkpointing: ActivationCheckpointing = ActivationCheckpointing.SELECTIVE
    selective_save_ops: tuple[str, ...] = ATTENTION_SAVE_OPS
    # Accepted for recipe compatibility; kernels here are hand-written, nothing is traced.
    compile: bool = True
    compile_dynamic: bool = False
    compile_options: Mapping[str, Any] = field(default_factory=dict)
    reduce_dtype: str = "float32"
    reshard_after_forward: bool = True
    # Not None: parameters created on the meta device get seeded N(0, 0.02) matrices, unit
    # norms and zero biases before the network's own post-materialisation rules run, so
    # synthetic recipes and benchmarks train from a well-defined state without a checkpoint.
    random_init_seed: int | None = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "activation_checkpointing",
                           ActivationCheckpointing(self.activation_checkpointing))
        for name in ("parameter_dtype", "reduce_dtype"):
            if not isinstance(getattr(torch, getattr(self, name), None), torch.dtype):
                raise ValueError(f"{name} must name a torch dtype, got {getattr(self, name)!r}")
        if self.context_parallel_size < 1:
            raise ValueError("context_parallel_size must be positive")
        if self.fsdp_mesh_shape is not None:
            object.__setattr__(self, "fsdp_mesh_shape", tuple(int(v) for v in self.fsdp_mesh_shape))
        object.__setattr__(self, "selective_save_ops", tuple(self.selective_save_ops))
        object.__setattr__(self, "compile_options", dict(self.compile_options))
        # Knobs of the reference's FSDP2 wrapping that this engine cannot honour are refused
        # rather than ignored.  (``reshard_after_forward`` is accepted in both settings: bf16
        # parameters stay whole on every GPU here, there is nothing to reshard; see
        # ``replicated_parameter_bytes`` for the memory this costs.)
        if self.reduce_dtype != "float32":
            raise ValueError("gradients are reduced in float32 by the peer-memory kernels; "
                             f"reduce_dtype={self.reduce_dtype!r} is not supported")
        shape = self.fsdp_mesh_shape
        if shape is not None and (len(shape) not in (1, 2) or any(v < 1 for v in shape)):
            raise ValueError(f"fsdp_mesh_shape must be (ranks,) or (nodes, ranks per node), got {shape}")
        if shape is not None and len(shape) == 2 and shape[1] > 8:
            raise ValueError("the optimizer state is sharded over the GPUs of one node (at most 8); "
                             f"fsdp_mesh_shape={shape} asks for a shard group of {shape[1]}")


def replicated_parameter_bytes(network: nn.Module, dtype: torch.dtype = torch.bfloat16) -> int:
    """Device memory that the whole parameters and gradients of ``network`` take on EVERY GPU:
    this engine shards the FP32 optimizer state (ZeRO-1/2), not the bf16 parameters, so a
    trainable tower costs 2 x its parameter bytes per GPU and a frozen one 1 x."""
    size = torch.empty((), dtype=dtype).element_size()
    total = 0
    for parameter in network.parameters():
        total += parameter.numel() * size * (2 if parameter.requires_grad else 1)
    return total


def _check_fits_replicated(network: nn.Module, dtype: torch.dtype, device: torch.device) -> None:
    """Fail before materialising a tower whose replicated parameters cannot fit the device
    (the sharded-parameter mode of FSDP2 would train it; this engine cannot)."""
    if device.type != "cuda":
        return
    need = replicated_parameter_bytes(network, dtype)
    free, _ = torch.cuda.mem_get_info(device)
    if need > free:
        raise MemoryError(
            f"{type(network).__name__}: whole parameters and gradients need {need / 2**30:.1f} GiB on every "
            f"GPU, {free / 2**30:.1f} GiB are free.  Parameters are replicated here (only the FP32 "
            "optimizer state is sharded); a model of this size needs parameter sharding, which this "
            "engine does not implement.")


_MESHES: dict[tuple, tuple[Any, Any]] = {}


def init_meshes(config: ParallelConfig, device_type: str):
    """Return ``(shard_mesh, cp_mesh)``; either may be ``None``.

    The shard mesh spans every rank (1-D, or ``(replicate, shard)`` across nodes).  The CP
    mesh is the inner dimension of a separate ``(world // cp, cp)`` mesh, so CP ranks are
    also shard ranks.
    """
    if not (dist.is_available() and dist.is_initialized()):
        return None, None
    from torch.distributed.device_mesh import init_device_mesh

    world = dist.get_world_size()
    local = get_local_world_size()
    shape = config.fsdp_mesh_shape
    if shape is None and config.fully_shard and 0 < local < world and world % local == 0:
        shape = (world // local, local)
    key = (device_type, world, config.fully_shard, config.context_parallel_size, shape)
    if key in _MESHES:
        return _MESHES[key]
    shard_mesh = None
    if config.fully_shard:
        shape = shape or (world,)
        if prod(shape) != world:
            raise ValueError(f"fsdp_mesh_shape {shape} does not cover {world} ranks")
        names = ("shard",) if len(shape) == 1 else ("replicate", "shard")
        shard_mesh = init_device_mesh(device_type, shape, mesh_dim_names=names)
    cp_mesh = None
    cp = config.context_parallel_size
    if cp > 1:
        if world % cp:
            raise ValueError(f"context_parallel_size {cp} does not divide {world} ranks")
        cp_mesh = init_device_mesh(device_type, (world // cp, cp),
                                   mesh_dim_names=("rest", "cp"))["cp"]
    _MESHES[key] = (shard_mesh, cp_mesh)
    return shard_mesh, cp_mesh


def _recomputes_itself(layer: nn.Module, args, kwargs) -> bool:
    """True when the call will take the fused CUDA layer, which keeps only the attention
    output and recomputes the rest in its own backward."""
    from agentgarten_b200.ops import fused_layer

    if len(args) < 3 or kwargs.get("time_embeddings") is not None or len(args) > 4 and args[4] is not None:
        return False
    try:
        return fused_layer.eligible(layer, args[0], args[2])
    except Exception:
        return False


class _KeepPlan:
    """Which layers of the operator-by-operator path keep their activations this pass.

    Recomputing a layer costs a third more compute and, under context parallelism, repeats
    its exchanges.  On a CUDA device the first layer of every pass therefore measures the free
    memory and the layers that fit (minus the reserve of ``AGB200_ACTIVATION_RESERVE_GB``) run
    without recomputation, the rest under it; ``AGB200_KEEP_ACTIVATIONS=never|always`` fixes
    the choice.  Ranks that share a clip take the minimum over their group, so that all of
    them issue the same collectives.
    """

    def __init__(self, group=None) -> None:
        self.group = group
        self.kept_layers = 0

    def keeps(self, layer: nn.Module, args) -> bool:
        from agentgarten_b200.ops import fused_layer

        mode = fused_layer._KEEP_MODE
        chunks = args[0]
        index = args[3] if len(args) > 3 else None
        if mode == "never" or index is None or not chunks[0].is_cuda:
            return False
        if mode == "always":
            return True
        if index == 0:
            self.kept_layers = self._budget(layer, chunks)
        return index < self.kept_layers

    def _budget(self, layer: nn.Module, chunks) -> int:
        from agentgarten_b200.ops import fused_layer

        device = chunks[0].device
        rows = sum(c.shape[0] * c.shape[1] for c in chunks)
        hidden = chunks[0].shape[-1]
        inner = layer.mlp_moe_gen.gate_proj.weight.shape[0]
        heads = (layer.num_attention_heads + 2 * layer.num_key_value_heads) * layer.head_dim
        # what autograd saves for one layer, operator by operator (bf16), with headroom for
        # the exchanged copies under context parallelism
        per_layer = int(rows * (8 * hidden + 4 * inner + 6 * heads) * 2 * 1.25)
        free, _ = torch.cuda.mem_get_info(device)
        free += torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        fit = max(0, int((free - fused_layer._RESERVE_BYTES) // max(per_layer, 1)))
        if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            agreed = torch.tensor([fit], device=device, dtype=torch.int64)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.group)
            fit = int(agreed.item())
        return fit


def _install_recompute(layer: nn.Module, plan: _KeepPlan | None = None) -> None:
    """Make ``layer(...)`` run under activation recomputation whenever grad is enabled and the
    plan does not keep the layer's activations.

    Only the bound ``forward`` of the instance is replaced, so module names and state-dict
    keys stay exactly those of the plain layer.
    """
    if getattr(layer, "_agb_recompute", False):
        return
    inner = layer.forward

    def forward(*args, **kwargs):
        if not torch.is_grad_enabled() or _recomputes_itself(layer, args, kwargs):
            return inner(*args, **kwargs)
        if plan is not None and plan.keeps(layer, args):
            return inner(*args, **kwargs)
        return checkpoint(inner, *args, use_reentrant=False, preserve_rng_state=True, **kwargs)

    layer.forward = forward
    layer._agb_recompute = True


def parallelize_network(network: ParallelNetwork, config: ParallelConfig, device):
    """Place ``network`` and return its context-parallel mesh (or ``None``)."""
    device = torch.device(device)
    dtype = getattr(torch, config.parameter_dtype)
    on_meta = any(p.is_meta for p in network.parameters())
    if on_meta:
        network.to(dtype=dtype)
    else:
        network.to(device=device, dtype=dtype)
    shard_mesh, cp_mesh = init_meshes(config, device.type)
    if cp_mesh is not None:
        network.enable_context_parallel(cp_mesh)
    mode = config.activation_checkpointing
    network.activation_checkpointing = mode
    if mode is not ActivationCheckpointing.NONE:
        # The fused CUDA layer keeps attention outputs and recomputes the rest by itself
        # (= "selective"); the op-by-op path recomputes the whole layer.
        plan = _KeepPlan(cp_mesh.get_group() if cp_mesh is not None else None)
        for layer in network.layers:
            _install_recompute(layer, plan)
    network.shard_mesh = shard_mesh
    network.parallel_config = config
    if on_meta:
        _check_fits_replicated(network, dtype, device)
        network.to_empty(device=device)
        if config.random_init_seed is not None:
            _random_init(network, int(config.random_init_seed))
        network.initialize_after_materialization()
    return cp_mesh


@torch.no_grad()
def _random_init(network: torch.nn.Module, seed: int) -> None:
    """The same values on every rank and device: drawn on the CPU, one parameter at a time."""
    generator = torch.Generator().manual_seed(seed)
    for name, p in network.named_parameters():
        if p.ndim >= 2 or not ("norm" in name or name.endswith("bias")):
            p.copy_(torch.randn(p.shape, generator=generator) * 0.02)
        elif "norm" in name:
            p.fill_(1.0)
        else:
            p.zero_()
