"""Flat-buffer sharded optimizer engine (CUDA).

All parameters of an optimizer are moved into one flat bf16 buffer and their gradients into
a second one; the ``nn.Parameter`` objects become views, so modules, autograd and state
dicts are unaffected.  With more than one rank both buffers are allocated as symmetric
memory, which gives every rank a pointer to every other rank's copy over NVLink.

Ownership follows the FSDP2 rule — rank ``r`` owns chunk ``r`` of ``torch.chunk(param,
world, dim=0)`` of every parameter — so the FP32 state a rank holds (master weights and
both moments of its chunks) has exactly the layout a ``Shard(0)`` DTensor of that parameter
would have, and sharded checkpoints are interchangeable with FSDP2 ones.

One update is two kernels (see ``csrc/zero.cu``):

1. ``zero_reduce`` — reads the owned ranges from *every* rank's gradient buffer (peer
   loads), averages in FP32, stores the FP32 shard and produces the squared norm and a
   non-finite flag.  The tiny all-reduce of those two numbers doubles as the point after
   which every rank may clear its gradient buffer.
2. ``zero_adam`` — Adam on the owned ranges with the clip coefficient applied on the fly,
   writing the new bf16 values straight into every rank's parameter buffer (peer stores).

Parity: replaces FSDP2's reduce-scatter + all-gather and Transformer-Engine's multi-tensor
Adam of the reference (``wm/infra/parallel.py:232-249``, ``wm/infra/optim/fused_adam.py:269-337``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from agentgarten_b200.ops import native

__all__ = ["ShardInfo", "ZeroEngine"]

UNIT = 16384      # elements per work unit
ALIGN = 64        # every parameter starts at a multiple of this many elements


@dataclass(frozen=True)
class ShardInfo:
    """Where this rank's chunk of a parameter sits."""

    global_shape: tuple[int, ...]
    row_offset: int        # first dim-0 row owned by this rank
    rows: int              # dim-0 rows owned (0 if none)
    flat_offset: int       # element offset of the chunk in the flat parameter buffer
    state_offset: int      # element offset of the chunk in the FP32 shard buffers
    numel: int


def _world(group) -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


_NODE_GROUPS: dict[tuple[int, int], tuple[Any, Any]] = {}


def node_groups(local_size: int) -> tuple[Any, Any]:
    """``(shard group, replica group)`` of a job that spans several nodes.

    Peer memory ends at the node, so the optimizer state is sharded over the ranks of a node
    (consecutive global ranks) and replicated across nodes; gradients are averaged across the
    replicas (ranks with the same local index) by NCCL before the node-local reduce.  This is
    the hybrid sharding of the reference (mesh ``(nodes, local)``, ``wm/infra/parallel.py:125-161``).
    Every rank must call this with the same ``local_size`` (groups are created collectively).
    """
    world, rank = dist.get_world_size(), dist.get_rank()
    key = (world, local_size)
    if key not in _NODE_GROUPS:
        if world % local_size:
            raise ValueError(f"{world} ranks do not split into nodes of {local_size}")
        shard = replica = None
        for node in range(world // local_size):
            members = list(range(node * local_size, (node + 1) * local_size))
            group = dist.new_group(members)
            if rank in members:
                shard = group
        for local in range(local_size):
            members = list(range(local, world, local_size))
            group = dist.new_group(members)
            if rank in members:
                replica = group
        _NODE_GROUPS[key] = (shard, replica)
    return _NODE_GROUPS[key]


class ZeroEngine:
    def __init__(self, optimizer: torch.optim.Optimizer, process_group: Any = None) -> None:
        self.optimizer = optimizer
        self.replica_group = None
        if process_group is None and dist.is_available() and dist.is_initialized():
            from agentgarten_b200.infra.distributed import get_local_world_size

            local = get_local_world_size()
            if 0 < local < dist.get_world_size():
                process_group, self.replica_group = node_groups(local)
        self.group = process_group
        self.world, self.rank = _world(process_group)
        if self.world > 8:
            raise ValueError("the peer-memory optimizer spans one node (at most 8 ranks)")
        self.C = native.require()
        groups = optimizer.param_groups
        params = [p for g in groups for p in g["params"]]
        if not params:
            raise ValueError("optimizer has no parameters")
        self.device = params[0].device
        self.params = params
        self.group_of = {id(p): gi for gi, g in enumerate(groups) for p in g["params"]}

        # ---- flat layout ------------------------------------------------------------
        offsets, total = [], 0
        for p in params:
            offsets.append(total)
            total += -(-p.numel() // ALIGN) * ALIGN
        self.total = total
        self.flat_param, self.param_ptrs = self._allocate(total)
        self.flat_grad, self.grad_ptrs = self._allocate(total)
        self.flat_grad.zero_()
        self.info: dict[int, ShardInfo] = {}
        units: list[tuple[int, int, int, int]] = []
        state_total = 0
        with torch.no_grad():
            for p, off in zip(params, offsets):
                view = self.flat_param[off: off + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.flat_grad[off: off + p.numel()].view(p.shape)
                shape = tuple(p.shape)
                rows_total = shape[0] if shape else 1
                row_elems = p.numel() // max(rows_total, 1) if p.numel() else 0
                chunk = -(-rows_total // self.world) if rows_total else 0
                first = min(self.rank * chunk, rows_total)
                rows = max(0, min(rows_total, first + chunk) - first)
                count = rows * row_elems
                state_offset = -(-state_total // 8) * 8
                self.info[id(p)] = ShardInfo(shape, first, rows, off + first * row_elems,
                                             state_offset, count)
                gi = self.group_of[id(p)]
                for start in range(0, count, UNIT):
                    units.append((off + first * row_elems + start, state_offset + start,
                                  min(UNIT, count - start), gi))
                state_total = state_offset + count
        self.state_total = max(state_total, 8)
        dev = self.device
        self.units = torch.tensor(units or [(0, 0, 0, 0)], dtype=torch.int64, device=dev)
        self.num_units = len(units)
        if not units:
            self.units = self.units[:0]
        # The averaged FP32 gradient shard is not materialised: the Adam kernel sums the
        # peers' gradients again (in the same order), which saves 4 bytes per owned element.
        self.gshard = None
        self.master = torch.zeros(self.state_total, dtype=torch.float32, device=dev)
        need_m = any(float(g["betas"][0]) > 0 for g in groups)
        need_v = any(float(g["betas"][1]) > 0 for g in groups)
        self.exp_avg = torch.zeros(self.state_total if need_m else 8, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.state_total if need_v else 8, dtype=torch.float32, device=dev)
        with torch.no_grad():
            for p in params:
                info = self.info[id(p)]
                if info.numel:
                    src = self.flat_param[info.flat_offset: info.flat_offset + info.numel]
                    self.master[info.state_offset: info.state_offset + info.numel].copy_(src.float())
        self.stats = torch.zeros(2, dtype=torch.float32, device=dev)   # sumsq, non-finite
        self.hyper_host = torch.zeros(len(groups), 8, dtype=torch.float32).pin_memory()
        self.hyper = torch.zeros(len(groups), 8, dtype=torch.float32, device=dev)
        self.scale = torch.ones(1, dtype=torch.float32, device=dev)
        self.steps = [0] * len(groups)
        self.skip_nonfinite = True
        self._reduced = False

    # ------------------------------------------------------------------ allocation
    def _allocate(self, numel: int) -> tuple[torch.Tensor, list[int]]:
        if self.world == 1:
            buf = torch.empty(numel, dtype=torch.bfloat16, device=self.device)
            return buf, [buf.data_ptr()]
        import torch.distributed._symmetric_memory as symm

        buf = symm.empty(numel, dtype=torch.bfloat16, device=self.device)
        group = self.group if self.group is not None else dist.group.WORLD
        handle = symm.rendezvous(buf, group=group)
        ptrs = [int(x) for x in handle.buffer_ptrs]
        self._handles = getattr(self, "_handles", []) + [handle]
        return buf, ptrs

    def _sync(self) -> None:
        """Stream-ordered rendezvous of all ranks (a one-element all-reduce)."""
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    @property
    def _token(self) -> torch.Tensor:
        if not hasattr(self, "_token_buf"):
            self._token_buf = torch.zeros(1, dtype=torch.float32, device=self.device)
        return self._token_buf

    # ------------------------------------------------------------------- gradients
    def reduce_gradients(self) -> None:
        if self._reduced:
            return
        if self.replica_group is not None:
            # across nodes first: every node then holds the job-wide average of its local index
            dist.all_reduce(self.flat_grad, op=dist.ReduceOp.AVG, group=self.replica_group)
        self._sync()  # every rank has finished writing its gradients
        self.C.zero_reduce(self.grad_ptrs, self.units, self.gshard, self.stats)
        native.count(2)
        if self.world > 1:
            # norm/flag over shards; after it every rank has finished reading peers' gradients
            dist.all_reduce(self.stats, group=self.group)
        self._reduced = True

    def grad_norm_sq(self) -> torch.Tensor:
        self.reduce_gradients()
        return self.stats[0]

    def found_nonfinite(self) -> torch.Tensor:
        self.reduce_gradients()
        return (self.stats[1] > 0).float()

    def zero_grad(self) -> None:
        self.flat_grad.zero_()
        self._reduced = False
        for p in self.params:
            if p.grad is None or p.grad.data_ptr() != self._grad_view_ptr(p):
                info_off = self._offset_of(p)
                p.grad = self.flat_grad[info_off: info_off + p.numel()].view(p.shape)

    def _offset_of(self, p: torch.Tensor) -> int:
        return (p.data_ptr() - self.flat_param.data_ptr()) // 2

    def _grad_view_ptr(self, p: torch.Tensor) -> int:
        return self.flat_grad.data_ptr() + 2 * self._offset_of(p)

    # ------------------------------------------------------------------------ step
    def step(self, grad_scale: float | torch.Tensor = 1.0) -> None:
        self.reduce_gradients()
        host = self.hyper_host
        for gi, g in enumerate(self.optimizer.param_groups):
            self.steps[gi] += 1
            t = self.steps[gi]
            b1, b2 = float(g["betas"][0]), float(g["betas"][1])
            correct = bool(g.get("bias_correction", True))
            host[gi, 0] = float(g["lr"])
            host[gi, 1], host[gi, 2] = b1, b2
            host[gi, 3] = float(g["eps"])
            host[gi, 4] = float(g["weight_decay"])
            host[gi, 5] = (1.0 - b1 ** t) if correct else 1.0
            host[gi, 6] = math.sqrt(1.0 - b2 ** t) if (correct and b2 > 0) else 1.0
            host[gi, 7] = 1.0 if self.optimizer.adam_w_mode else 0.0
        self.hyper.copy_(host, non_blocking=True)
        if isinstance(grad_scale, torch.Tensor):
            self.scale.copy_(grad_scale.reshape(1).to(self.scale.dtype))
        else:
            self.scale.fill_(float(grad_scale))
        skip = self.stats[1:2] if self.skip_nonfinite else None
        self.C.zero_adam(self.param_ptrs, self.grad_ptrs, self.units, self.gshard, self.master, self.exp_avg,
                         self.exp_avg_sq, self.hyper, self.scale, skip)
        native.count()
        self._sync()  # every rank's parameter buffer is complete before the next forward
        self._reduced = False

    # --------------------------------------------------------------- state exchange
    def _views(self, p: torch.Tensor) -> dict[str, torch.Tensor]:
        info = self.info[id(p)]
        # a zero-dimensional parameter lives whole on the first rank and is empty elsewhere
        shape = (info.rows, *info.global_shape[1:]) if info.global_shape else (() if info.numel else (0,))
        lo, hi = info.state_offset, info.state_offset + info.numel
        g = self.optimizer.param_groups[self.group_of[id(p)]]
        out = {"master_param": self.master[lo:hi].view(shape)}
        if float(g["betas"][0]) > 0:
            out["exp_avg"] = self.exp_avg[lo:hi].view(shape)
        if float(g["betas"][1]) > 0:
            out["exp_avg_sq"] = self.exp_avg_sq[lo:hi].view(shape)
        return out

    def publish_state(self) -> None:
        """Expose the shard state through ``optimizer.state`` (views, no copies)."""
        for p in self.params:
            state = self.optimizer.state[p]
            state["step"] = torch.tensor(float(self.steps[self.group_of[id(p)]]))
            state.update(self._views(p))

    def adopt_state(self) -> None:
        """Copy state loaded into ``optimizer.state`` back into the flat shard buffers.

        Accepts either this rank's chunk or the full tensor of a parameter."""
        for p in self.params:
            state = self.optimizer.state.get(p)
            if not state:
                continue
            info = self.info[id(p)]
            if "step" in state:
                self.steps[self.group_of[id(p)]] = int(float(state["step"]))
            views = self._views(p)
            for key, view in views.items():
                value = state.get(key)
                if not isinstance(value, torch.Tensor) or value.data_ptr() == view.data_ptr():
                    continue
                if hasattr(value, "to_local"):
                    value = value.to_local()
                if tuple(value.shape) == info.global_shape and info.global_shape:
                    value = value[info.row_offset: info.row_offset + info.rows]
                if view.numel() == 0:
                    state[key] = view
                    continue
                view.copy_(value.to(view.device, torch.float32).reshape(view.shape))
                state[key] = view

    def refresh_master(self) -> None:
        """Re-derive FP32 master weights from the bf16 parameters (after loading weights)."""
        with torch.no_grad():
            for p in self.params:
                info = self.info[id(p)]
                if info.numel:
                    src = self.flat_param[info.flat_offset: info.flat_offset + info.numel]
                    self.master[info.state_offset: info.state_offset + info.numel].copy_(src.float())
