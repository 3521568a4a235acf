"""Tensor-parallel serving of the generation tower over NVLink peer memory.

Megatron-style sharding with a row-sharded residual stream: attention heads and MLP columns
are split over the ranks; the residual stream is owned in tiles of 128 rows (tile ``t``
belongs to rank ``t % world``).  Per layer and rank the kernels are

1. ``QKV = X @ Wqkv_local^T`` — the tcgen05 GEMM whose TMA producer waits, tile by tile, for
   rows of ``X`` that their owners push into this GPU's memory (all-gather fused into the
   GEMM);
2. per-head RMSNorm + RoPE, attention over the local heads and the local slice of the KV
   cache (no communication);
3. ``partial = attn @ Wo_local^T`` — the GEMM whose epilogue stores each output tile straight
   into the partial-sum slot of the tile's owner through the peer mapping and bumps the
   owner's arrival counter (reduce-scatter fused into the GEMM);
4. on the owner: wait for ``world`` partials, add them to the residual rows, RMSNorm, and
   store the normalised rows into every rank's ``X`` (the next all-gather), all in one
   kernel;
5. the same pattern for gate/up (column parallel, SiLU·mul local) and down (row parallel).

Counters are monotonic and use numbers live in device memory, so the launch sequence of a
step is captured once in a CUDA graph and replayed.  Every wait is bounded: a rank that
does not arrive makes the others record ``kTimeoutPeer`` in the status word and return.
With one rank the same kernels run against the local buffers.

Parity: the reference serves on one GPU only (``wm/inference/serving.py:17-96``); this is
the multi-GPU counterpart of its ``project`` / ``finish`` halves
(``wm/networks/cosmos3/layers.py:269-312``).
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from agentgarten_b200 import ops
from agentgarten_b200.ops import native

__all__ = ["TensorParallelServing"]

_TILE = 128
_COLUMN_TILE = 256


class TensorParallelServing:
    def __init__(self, network: torch.nn.Module, group: dist.ProcessGroup | None = None, *,
                 max_tokens: int = 8192) -> None:
        config = network.config
        if config.timestep_conditioning != "add":
            raise ValueError("tensor-parallel serving supports additive timestep conditioning only")
        self.network = network
        self.group = group
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
        if kv_heads % self.world or config.intermediate_size % (self.world * 8):
            raise ValueError(f"{self.world} ranks do not divide {kv_heads} KV heads / the MLP width")
        self.heads, self.kv_heads, self.dim = heads // self.world, kv_heads // self.world, config.head_dim
        self.hidden = config.hidden_size
        self.inner = config.intermediate_size // self.world
        self.eps = config.rms_norm_eps
        self.device = next(network.parameters()).device
        self.max_tiles = -(-max_tokens // _TILE)
        self.max_owned = -(-self.max_tiles // self.world)
        self.kv_slice = slice(self.rank * self.kv_heads, (self.rank + 1) * self.kv_heads)
        self._shard_weights()
        self._allocate()
        # Rows per CTA of the reduce kernel: 0 lets the kernel choose from the rows a rank owns.
        self.reduce_rows = 0
        # Set to a dict to collect (start, stop) CUDA events per phase of run() (eager mode only).
        self.trace: dict[str, list] | None = None

    def _mark(self, phase: str, start: torch.cuda.Event | None = None):
        """Phase timing for diagnosis: returns a started event, or closes one under ``phase``."""
        if self.trace is None or torch.cuda.is_current_stream_capturing():
            return None
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        if start is not None:
            self.trace.setdefault(phase, []).append((start, event))
        return event

    def trace_summary(self) -> dict[str, float]:
        """Mean milliseconds per phase call and calls per phase, from the collected events."""
        torch.cuda.synchronize(self.device)
        return {phase: sum(a.elapsed_time(b) for a, b in spans) / len(spans)
                for phase, spans in (self.trace or {}).items()}

    # ------------------------------------------------------------------------ set-up
    @torch.no_grad()
    def _shard_weights(self) -> None:
        r, d = self.rank, self.dim
        q_rows = slice(r * self.heads * d, (r + 1) * self.heads * d)
        kv_rows = slice(r * self.kv_heads * d, (r + 1) * self.kv_heads * d)
        mlp_rows = slice(r * self.inner, (r + 1) * self.inner)
        self.layers = []
        for layer in self.network.layers:
            to_q, to_k, to_v, to_out, norm_q, norm_k = layer.self_attn.parts()
            if to_q.bias is not None:
                raise ValueError("tensor-parallel serving expects bias-free attention projections")
            mlp = layer.mlp_moe_gen
            self.layers.append({
                "qkv": torch.cat((to_q.weight[q_rows], to_k.weight[kv_rows], to_v.weight[kv_rows])).contiguous(),
                "out": to_out.weight[:, q_rows].contiguous(),
                "gate_up": torch.cat((mlp.gate_proj.weight[mlp_rows], mlp.up_proj.weight[mlp_rows])).contiguous(),
                "down": mlp.down_proj.weight[:, mlp_rows].contiguous(),
                "norm_q": norm_q.weight, "norm_k": norm_k.weight, "head_eps": norm_q.variance_epsilon,
                "norm_in": layer.input_layernorm_moe_gen.weight,
                "norm_mid": layer.post_attention_layernorm_moe_gen.weight,
            })

    def _symmetric(self, numel: int, dtype: torch.dtype, data: bool = False) -> tuple[torch.Tensor, list[int]]:
        """A buffer every rank can address.  Counters start at zero; ``data`` buffers (rows that
        peers push) start at zero too, or as NaN under ``AGB200_POISON=1`` so that a consumer that
        reads a row nobody pushed produces non-finite values instead of plausible ones."""
        from .debug import poison

        if self.world == 1:
            buf = torch.zeros(numel, dtype=dtype, device=self.device)
            if data:
                poison(buf)
            return buf, [buf.data_ptr()]
        import torch.distributed._symmetric_memory as symm

        buf = symm.empty(numel, dtype=dtype, device=self.device)
        buf.zero_()
        if data:
            poison(buf)
        handle = symm.rendezvous(buf, group=self.group if self.group is not None else dist.group.WORLD)
        self._handles.append(handle)
        return buf, [int(p) for p in handle.buffer_ptrs]

    def _allocate(self) -> None:
        self._handles: list = []
        h = self.hidden
        self.x, self.x_ptrs = self._symmetric(self.max_tiles * _TILE * h, torch.bfloat16, data=True)
        self.slots, self.slot_ptrs = self._symmetric(self.world * self.max_owned * _TILE * h, torch.bfloat16,
                                                     data=True)
        counters, pointers = self._symmetric(self.max_tiles + self.max_owned + 1, torch.int32)
        self.ready = counters[: self.max_tiles]
        self.arrive = counters[self.max_tiles: self.max_tiles + self.max_owned]
        self.done = counters[self.max_tiles + self.max_owned:]
        self.ready_ptrs = list(pointers)
        self.arrive_ptrs = [p + 4 * self.max_tiles for p in pointers]
        self.done_ptrs = [p + 4 * (self.max_tiles + self.max_owned) for p in pointers]
        self.hidden_own = torch.zeros(self.max_owned * _TILE, h, dtype=torch.bfloat16, device=self.device)
        # consumed amounts of the ready / arrival counters, completed steps, last-CTA tickets
        self.state = torch.zeros(self.max_tiles + self.max_owned + 3, dtype=torch.int32, device=self.device)
        self.x_seen = self.state[: self.max_tiles]
        self.slot_seen = self.state[self.max_tiles: self.max_tiles + self.max_owned]
        tail = self.state[self.max_tiles + self.max_owned:]
        self.steps, self.gemm_ticket, self.reduce_ticket = tail[0:1], tail[1:2], tail[2:3]
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # zeroed counters everywhere before the first push

    # --------------------------------------------------------------------------- step
    def _reduce(self, m: int, owned: int, weight: torch.Tensor, seed: torch.Tensor | None) -> None:
        native.count()
        native.ext().tp_reduce_norm(
            self.rank, self.world, m, self.slots, self.arrive, self.slot_seen, self.reduce_ticket,
            4 * -(-self.hidden // _COLUMN_TILE), self.hidden_own, seed, weight, self.eps,
            self.x_ptrs, self.ready_ptrs, owned, self.done, self.steps, self.reduce_rows)

    def _gather_gemm(self, x: torch.Tensor, weight: torch.Tensor, *, close: bool) -> torch.Tensor:
        out = torch.empty(x.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        native.count()
        native.ext().tp_gemm(x, weight, out, self.rank, self.world, self.ready, self.x_seen,
                             self.gemm_ticket if close else None, [], [], 0)
        return out

    def _scatter_gemm(self, a: torch.Tensor, weight: torch.Tensor, owned: int) -> None:
        native.count()
        native.ext().tp_gemm(a, weight, None, self.rank, self.world, None, None, None,
                             self.slot_ptrs, self.arrive_ptrs, owned)

    @torch.no_grad()
    def run(self, tokens: torch.Tensor, rope: tuple[torch.Tensor, torch.Tensor],
            attend: Callable[[int, list, list, list], list]) -> torch.Tensor:
        """``tokens`` ``[1, M, H]`` (identical on every rank) through all layers and the head.

        Returns ``proj_out(norm(hidden))`` for every token, ``[1, M, out]``, complete on every
        rank.  ``attend(index, [q], [k], [v])`` sees this rank's heads only.
        """
        if tokens.shape[0] != 1:
            raise ValueError("tensor-parallel serving runs one stream (batch 1)")
        m = tokens.shape[1]
        tiles = -(-m // _TILE)
        if tiles > self.max_tiles:
            raise ValueError(f"{m} tokens exceed the buffers sized at construction")
        owned = -(-tiles // self.world)
        cos, sin = rope
        x = self.x[: m * self.hidden].view(m, self.hidden)
        q_cols, kv_cols = self.heads * self.dim, self.kv_heads * self.dim
        layers = self.layers
        self._reduce(m, owned, layers[0]["norm_in"], tokens.reshape(m, self.hidden).contiguous())
        for index, w in enumerate(layers):
            t0 = self._mark("")
            qkv = self._gather_gemm(x, w["qkv"], close=True)
            t1 = self._mark("gather+qkv gemm", t0)
            # the head-norm kernel reads its column block of the fused product in place
            C = native.ext()
            native.count(2)
            q, _ = C.head_norm_rope_fwd(qkv[:, :q_cols].view(1, m, self.heads, self.dim), w["norm_q"],
                                        cos, sin, w["head_eps"])
            k, _ = C.head_norm_rope_fwd(qkv[:, q_cols:q_cols + kv_cols].view(1, m, self.kv_heads, self.dim),
                                        w["norm_k"], cos, sin, w["head_eps"])
            v = qkv[:, q_cols + kv_cols:].view(1, m, self.kv_heads, self.dim)  # copied into the cache as is
            t2 = self._mark("head norm + rope", t1)
            (mixed,) = attend(index, [q], [k], [v])
            t3 = self._mark("cache write + attention", t2)
            self._scatter_gemm(mixed.reshape(m, q_cols), w["out"], owned)
            t4 = self._mark("out gemm + scatter", t3)
            self._reduce(m, owned, w["norm_mid"], None)
            t5 = self._mark("reduce + norm + push", t4)
            both = self._gather_gemm(x, w["gate_up"], close=True)  # [m, gate columns | up columns]
            t6 = self._mark("gather+gate/up gemm", t5)
            native.count()
            act = native.ext().silu_mul_pair(both)
            t7 = self._mark("silu mul", t6)
            self._scatter_gemm(act, w["down"], owned)
            t8 = self._mark("down gemm + scatter", t7)
            following = layers[index + 1]["norm_in"] if index + 1 < len(layers) \
                else self.network.norm_moe_gen.weight
            self._reduce(m, owned, following, None)
            self._mark("reduce + norm + push", t8)
        # The head reads the gathered, normalised rows (and closes this use of X); the end of
        # the step is then announced to every rank, whose next step overwrites X here.
        head = self.network.proj_out
        patches = self._gather_gemm(x, head.weight, close=True)
        native.count()
        native.ext().tp_signal_done(self.done_ptrs, self.state)
        if head.bias is not None:
            patches = patches + head.bias
        return patches.view(1, m, -1)
