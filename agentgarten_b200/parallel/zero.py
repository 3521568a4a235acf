"""Flat-buffer sharded optimizer engine (CUDA).

All parameters of an optimizer are moved into one flat bf16 buffer and their gradients into
a second one; the ``nn.Parameter`` objects become views, so modules, autograd and state
dicts are unaffected.  With more than one rank both buffers are allocated as symmetric
memory, which gives every rank a pointer to every other rank's copy over NVLink.

Ownership follows the FSDP2 rule — rank ``r`` owns chunk ``r`` of ``torch.chunk(param,
world, dim=0)`` of every parameter — so the FP32 state a rank holds (master weights and
both moments of its chunks) has exactly the layout a ``Shard(0)`` DTensor of that parameter
would have, and sharded checkpoints are interchangeable with FSDP2 ones.

One update (see ``csrc/zero.cu``):

1. ``zero_reduce_range`` per *bucket* — reads the owned ranges of a bucket from every rank's
   gradient buffer (peer loads), averages in FP32, stores the FP32 shard and per-CTA partial
   sums of squares.  The fused generation layers report "the gradients of my parameters are
   complete" from their backward pass (:func:`grads_ready`); the engine then announces the
   bucket to the peers (a system-scope counter, ``zero_signal``) and launches its reduce on a
   side stream, where it waits for the peers' announcements and runs under the backward pass
   of the earlier layers.  Gradients cross NVLink once.
2. ``zero_stats`` — folds the partial sums in a fixed order and exchanges the two numbers
   (squared norm, non-finite flag) through the ranks' slot tables: the global norm without a
   library collective, and the point after which every rank may clear its gradient buffer.
3. ``zero_adam`` — Adam on the owned ranges from the averaged gradient (written back in bf16
   over this rank's own gradient of those ranges by the reduce) with the clip
   coefficient applied on the fly, writing the new bf16 values straight into every rank's
   parameter buffer (peer stores); a "done" counter then tells the peers that their buffers
   are complete.

Parity: replaces FSDP2's reduce-scatter + all-gather and Transformer-Engine's multi-tensor
Adam of the reference (``wm/infra/parallel.py:232-249``, ``wm/infra/optim/fused_adam.py:269-337``).
"""

from __future__ import annotations

import math
import os
import weakref
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from agentgarten_b200.ops import native

__all__ = ["ShardInfo", "ZeroEngine", "arm_overlap", "grads_ready", "note_forward"]

# Live engines, for the module-level hooks below.  An engine keeps its parameters alive, so
# the ids in its ``param_units`` cannot be reused by other tensors while it is in this set.
_ENGINES: "weakref.WeakSet[ZeroEngine]" = weakref.WeakSet()


def arm_overlap(armed: bool = True) -> None:
    """Tell every engine that the backward pass about to run is the last of its update."""
    for engine in list(_ENGINES):
        engine.arm_overlap(armed)


def _owner(params):
    for engine in list(_ENGINES):
        if params and id(params[0]) in engine.param_units:
            return engine
    return None


def note_forward(params) -> None:
    """A layer whose backward pass will report through :func:`grads_ready` ran its forward
    pass on ``params``: one more backward pass must finish before its bucket is complete."""
    if _ENGINES:
        params = tuple(params)
        engine = _owner(params)
        if engine is not None:
            engine._pending[id(params[0])] = engine._pending.get(id(params[0]), 0) + 1


def grads_ready(params) -> None:
    """A backward pass of one layer has written its gradients of ``params``.  When it was the
    last outstanding one of that layer in this update, the layer's bucket is reduced."""
    if _ENGINES:
        params = tuple(params)
        engine = _owner(params)
        if engine is not None:
            left = engine._pending.get(id(params[0]), 1) - 1
            engine._pending[id(params[0])] = left
            if left <= 0:
                engine.grads_ready(params)

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
        self.param_units: dict[int, tuple[int, int]] = {}  # parameter -> [first, last) unit
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
                self.param_units[id(p)] = (len(units), len(units) + -(-count // UNIT))
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
        # No FP32 gradient shard: with peers the reduce writes the bf16 average back over this
        # rank's own gradient of the ranges it owns (which no peer reads), Adam then reads only
        # local memory and the peers' gradients cross NVLink once.
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
        # ---- bucketed reduce: partial sums, counters, side stream ---------------------------
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self._full_parts = max(1, min(self.num_units, sms * 8))
        # CTAs of a bucket reduced under the backward pass: one per SM, so that the burst is
        # short (bound by NVLink, a fraction of a millisecond per layer) and slows every SM's
        # resident GEMM or attention CTA alike instead of stretching the kernels' slowest SM.
        self._bucket_parts = sms
        self._max_buckets = 64
        self.partial_sumsq = torch.zeros(self._max_buckets * self._bucket_parts + self._full_parts,
                                         dtype=torch.float32, device=dev)
        self.partial_bad = torch.zeros_like(self.partial_sumsq, dtype=torch.int32)
        self._buckets: dict[tuple[int, int], int] = {}   # unit range -> slot (same on all ranks)
        self._launched: list[tuple[int, int]] = []       # ranges reduced so far in this update
        self._used_parts = 0
        self._armed = False
        self._pending: dict[int, int] = {}   # first parameter of a layer -> backward passes outstanding
        self._epoch = 0
        self._side = torch.cuda.Stream(device=dev)
        self.counter_ptrs: list[int] = []
        self.table_ptrs: list[int] = []
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm

            group = self.group if self.group is not None else dist.group.WORLD
            self.counters = symm.empty(128, dtype=torch.int32, device=dev)   # 0..95 buckets, 96.. tails, 127 done
            self.table = symm.empty(32, dtype=torch.int32, device=dev)       # [8 ranks][sum, flag, epoch, -]
            self.counters.zero_()
            self.table.zero_()
            for buf in (self.counters, self.table):
                handle = symm.rendezvous(buf, group=group)
                self._handles.append(handle)
                (self.counter_ptrs if buf is self.counters else self.table_ptrs).extend(
                    int(x) for x in handle.buffer_ptrs)
            torch.cuda.synchronize(dev)
            dist.barrier(group=group)  # zeroed counters everywhere before the first signal
        _ENGINES.add(self)

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

    # ------------------------------------------------------------------- gradients
    def arm_overlap(self, armed: bool = True) -> None:
        """The next backward pass is the last one of this update: buckets reported through
        :func:`grads_ready` are reduced at once, under the rest of the backward pass."""
        self._armed = (bool(armed) and self.world > 1 and self.replica_group is None
                       and os.environ.get("AGB200_GRAD_OVERLAP", "1") != "0")

    def _launch_range(self, lo: int, hi: int, stream: torch.cuda.Stream, parts: int) -> None:
        """Announce units [lo, hi) to the peers and reduce them on ``stream``."""
        ready = slot = None
        target = 0
        if self.world > 1:
            key = (lo, hi)
            if key not in self._buckets:
                if len(self._buckets) >= 127:
                    raise RuntimeError("too many gradient buckets")
                self._buckets[key] = len(self._buckets)
            slot = self._buckets[key]
            ready, target = self.counters, self.world * self._epoch
        with torch.cuda.stream(stream):
            if slot is not None:
                self.C.zero_signal(self.counter_ptrs, slot, self.counters)
            self.C.zero_reduce_range(self.grad_ptrs, self.units, lo, hi, self.gshard, self.partial_sumsq,
                                     self.partial_bad, self._used_parts, parts, ready,
                                     slot if slot is not None else 0, target,
                                     self.rank if self.world > 1 else -1)
        native.count(2 if slot is not None else 1)
        self._used_parts += parts
        self._launched.append((lo, hi))

    def grads_ready(self, params) -> bool:
        """Called from a layer's backward pass when the gradients of ``params`` are complete on
        this rank.  Returns True when their reduce was launched (side stream)."""
        if not self._armed or self._reduced:
            return False
        ranges = [self.param_units[id(p)] for p in params if id(p) in self.param_units]
        if not ranges:
            return False
        lo, hi = min(r[0] for r in ranges), max(r[1] for r in ranges)
        if hi <= lo or sum(r[1] - r[0] for r in ranges) != hi - lo:
            return False  # not one contiguous run of units: left to the final reduce
        if any(lo < b and a < hi for a, b in self._launched) or len(self._launched) >= self._max_buckets:
            return False
        if not self._launched:
            self._epoch += 1
        self._side.wait_stream(torch.cuda.current_stream(self.device))
        self._launch_range(lo, hi, self._side, self._bucket_parts)
        return True

    def reduce_gradients(self) -> None:
        if self._reduced:
            return
        if self.replica_group is not None:
            # across nodes first: every node then holds the job-wide average of its local index
            dist.all_reduce(self.flat_grad, op=dist.ReduceOp.AVG, group=self.replica_group)
        main = torch.cuda.current_stream(self.device)
        if not self._launched:
            self._epoch += 1
        else:
            main.wait_stream(self._side)
        # what the backward pass did not report: the complement of the launched ranges
        cursor = 0
        for lo, hi in sorted(self._launched) + [(self.num_units, self.num_units)]:
            if lo > cursor:
                share = max(1, min(self._full_parts - 0, (lo - cursor)))
                share = min(share, self.partial_sumsq.numel() - self._used_parts)
                self._launch_range(cursor, lo, main, share)
            cursor = max(cursor, hi)
        self.C.zero_stats(self.partial_sumsq, self.partial_bad, self._used_parts,
                          self.table_ptrs, self.rank, self._epoch, self.stats)
        native.count()
        self._launched.clear()
        self._pending.clear()
        self._used_parts = 0
        self._armed = False
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
        # after the reduce this rank's own buffer holds the averaged gradient of its ranges
        self.C.zero_adam(self.param_ptrs, [self.grad_ptrs[self.rank]], self.units, self.gshard, self.master, self.exp_avg,
                         self.exp_avg_sq, self.hyper, self.scale, skip)
        native.count()
        if self.world > 1:
            # every rank's stores into this rank's parameter buffer are complete before the
            # next forward: each rank adds one to slot 127 of all tables after its Adam kernel
            self.C.zero_signal(self.counter_ptrs, 127, self.counters)
            self.C.zero_wait(self.counters, 127, self.world * self._epoch)
            native.count(2)
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
