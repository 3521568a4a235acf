"""Adam/AdamW with FP32 moments and optional FP32 master weights.

Two execution paths share one state layout (``step``, ``exp_avg``, ``exp_avg_sq``,
``master_param`` per parameter, all FP32):

* **flat / sharded (CUDA)** – parameters and gradients of the optimizer live in one flat
  bf16 buffer each; every rank owns the dim-0 chunk ``rank`` of every parameter (the FSDP2
  ownership rule) and holds FP32 state only for it.  ``reduce_gradients()`` runs the
  peer-memory reduce-scatter kernel (FP32 sum of all ranks' gradients, plus the squared
  norm and a non-finite flag as side outputs), ``step()`` runs the fused Adam kernel that
  also writes the new bf16 values into every peer's parameter buffer.  With one GPU the
  same two kernels run with a single peer.
* **foreach (CPU, or CUDA without the flat engine)** – the textbook update with
  ``torch._foreach`` ops; with a process group the gradients are averaged by all-reduce and
  the state stays replicated.

``beta1 == 0`` drops the first moment, ``beta2 == 0`` uses ``|g|`` as denominator.

Parity: reference ``wm/infra/optim/fused_adam.py:87-544`` (which dispatches to
Transformer-Engine's multi-tensor Adam on CUDA).
"""

from __future__ import annotations

from collections.abc import Iterable
from typing import Any

import torch
import torch.distributed as dist

__all__ = ["FusedAdam"]

_STATE_KEYS = ("exp_avg", "exp_avg_sq", "master_param")


def _f(value: Any) -> float:
    return float(value.item()) if isinstance(value, torch.Tensor) else float(value)


class FusedAdam(torch.optim.Optimizer):
    def __init__(self, params: Iterable[torch.Tensor] | Iterable[dict[str, Any]],
                 lr: float | torch.Tensor = 1e-3, *, bias_correction: bool = True,
                 betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-10,
                 adam_w_mode: bool = True, weight_decay: float = 0.0, amsgrad: bool = False,
                 use_te_capturable_kernel: bool = False, master_weights: bool = False,
                 process_group: Any = None, flat: bool | None = None) -> None:
        if amsgrad:
            raise ValueError("FusedAdam does not implement AMSGrad")
        if master_weights and not use_te_capturable_kernel:
            raise ValueError("FP32 master weights require use_te_capturable_kernel=True")
        defaults = {"lr": lr, "bias_correction": bias_correction, "betas": tuple(betas),
                    "eps": eps, "weight_decay": weight_decay}
        self._check_group(defaults)
        super().__init__(params, defaults)
        self.adam_w_mode = bool(adam_w_mode)
        self.use_te_capturable_kernel = bool(use_te_capturable_kernel)
        self.master_weights = bool(master_weights)
        self.process_group = process_group
        # Multiplier folded into the next update (gradient clipping sets it); device
        # scalar on the flat path so clipping needs no host synchronisation.
        self.grad_scale: float | torch.Tensor = 1.0
        self._engine = None
        every = [p for g in self.param_groups for p in g["params"]]
        if flat is None:
            flat = bool(every) and all(p.is_cuda and p.dtype == torch.bfloat16 for p in every)
        if flat:
            from agentgarten_b200.parallel.zero import ZeroEngine

            self._engine = ZeroEngine(self, process_group=process_group)

    # ------------------------------------------------------------------ validation
    @staticmethod
    def _check_group(group: dict[str, Any]) -> None:
        """Every hyper-parameter is one finite number (a Python scalar or a one-element tensor);
        rates, epsilon and decay are not negative, both betas lie in [0, 1).  The messages are the
        reference's (``wm/infra/optim/fused_adam.py:130-158``)."""
        import math

        def number(name: str, value: Any) -> float:
            if torch.is_tensor(value) and value.numel() != 1:
                raise ValueError(f"FusedAdam {name} must be a scalar")
            try:
                result = _f(value)
            except (TypeError, ValueError, OverflowError) as error:
                raise ValueError(f"FusedAdam {name} must be a finite scalar") from error
            if not math.isfinite(result):
                raise ValueError(f"FusedAdam {name} must be finite")
            return result

        for name in ("lr", "eps", "weight_decay"):
            if number(name, group[name]) < 0:
                raise ValueError(f"FusedAdam {name} must be non-negative")
        betas = group["betas"]
        if isinstance(betas, (str, bytes)) or not hasattr(betas, "__len__") or len(betas) != 2:
            raise ValueError("FusedAdam betas must contain two scalars")
        for position, beta in enumerate(betas, start=1):
            if not 0.0 <= number(f"beta{position}", beta) < 1.0:
                raise ValueError(f"FusedAdam beta{position} must be in [0, 1)")

    # ----------------------------------------------------------------------- state
    def _init_state(self, p: torch.Tensor, beta1: float, beta2: float) -> dict[str, Any]:
        state = self.state[p]
        if "step" not in state:
            state["step"] = torch.zeros((), dtype=torch.float32)
        if beta1 > 0:
            if "exp_avg" not in state:
                state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
        else:
            state.pop("exp_avg", None)
        if beta2 > 0:
            if "exp_avg_sq" not in state:
                state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        else:
            state.pop("exp_avg_sq", None)
        if self.master_weights and "master_param" not in state:
            state["master_param"] = p.detach().clone().float()
        return state

    @property
    def engine(self):
        """The flat sharded engine (``None`` on the foreach path)."""
        return self._engine

    # ------------------------------------------------------------------- gradients
    def reduce_gradients(self) -> None:
        """Combine gradients across data-parallel ranks (mean). Idempotent per update."""
        if self._engine is not None:
            self._engine.reduce_gradients()
            return
        if getattr(self, "_reduced", False):
            return
        group = self.process_group
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            world = dist.get_world_size(group)
            grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
            if grads:
                flat = torch.cat([g.reshape(-1).float() for g in grads])
                dist.all_reduce(flat, group=group)
                flat.div_(world)
                offset = 0
                for g in grads:
                    g.copy_(flat[offset: offset + g.numel()].view_as(g))
                    offset += g.numel()
        self._reduced = True

    def grad_norm_sq(self) -> torch.Tensor:
        """Squared L2 norm of the reduced gradient (device scalar)."""
        self.reduce_gradients()
        if self._engine is not None:
            return self._engine.grad_norm_sq()
        grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not grads:
            return torch.zeros(())
        norms = torch._foreach_norm(grads, 2.0)
        return torch.stack([n.float() for n in norms]).square().sum()

    def found_nonfinite(self) -> torch.Tensor | None:
        if self._engine is not None:
            return self._engine.found_nonfinite()
        return None

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._reduced = False
        if self._engine is not None:
            self._engine.zero_grad()
            return
        super().zero_grad(set_to_none=set_to_none)

    # ------------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            self._check_group(group)
        self.reduce_gradients()
        if self._engine is not None:
            self._engine.step(self.grad_scale)
        else:
            self._foreach_step()
        self.grad_scale = 1.0
        self._reduced = False
        return loss

    def _foreach_step(self) -> None:
        scale = _f(self.grad_scale)
        for group in self.param_groups:
            beta1, beta2 = (_f(b) for b in group["betas"])
            lr, eps, wd = _f(group["lr"]), _f(group["eps"]), _f(group["weight_decay"])
            correct = bool(group["bias_correction"])
            buckets: dict[int, list[tuple[torch.Tensor, dict[str, Any]]]] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("FusedAdam does not support sparse gradients")
                state = self._init_state(p, beta1, beta2)
                step = int(_f(state["step"])) + 1
                state["step"].fill_(step)
                if p.numel():
                    buckets.setdefault(step, []).append((p, state))
            for step, members in buckets.items():
                params = [p for p, _ in members]
                grads = [p.grad.float() * scale if scale != 1.0 else p.grad.float()
                         for p in params]
                masters = [s["master_param"] for _, s in members] if self.master_weights else []
                targets = masters or params
                if not self.adam_w_mode and wd:
                    grads = torch._foreach_add(grads, [t.float() for t in targets], alpha=wd)
                if beta1 > 0:
                    first = [s["exp_avg"] for _, s in members]
                    torch._foreach_lerp_(first, grads, 1.0 - beta1)
                    numer = first
                else:
                    numer = grads
                if beta2 > 0:
                    second = [s["exp_avg_sq"] for _, s in members]
                    torch._foreach_mul_(second, beta2)
                    torch._foreach_addcmul_(second, grads, grads, value=1.0 - beta2)
                    denom = torch._foreach_sqrt(second)
                else:
                    denom = [g.abs() for g in grads]
                c1 = 1.0 - beta1 ** step if correct else 1.0
                c2 = ((1.0 - beta2 ** step) ** 0.5 if beta2 > 0 else 1.0) if correct else 1.0
                torch._foreach_div_(denom, c2)
                torch._foreach_add_(denom, eps)
                if masters or all(t.dtype == torch.float32 for t in targets):
                    work = targets
                else:
                    work = [t.float() for t in targets]
                if self.adam_w_mode and wd:
                    torch._foreach_mul_(work, 1.0 - lr * wd)
                torch._foreach_addcdiv_(work, numer, denom, value=-lr / c1)
                if work is not params:
                    torch._foreach_copy_(params, work)

    # ------------------------------------------------------------------ state dict
    def state_dict(self) -> dict[str, Any]:
        if self._engine is not None:
            self._engine.publish_state()
        return super().state_dict()

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        super().load_state_dict(state_dict)
        # Moments and master weights stay FP32 regardless of the parameter dtype
        # (the base class casts floating state to the parameter's dtype).
        saved = state_dict.get("state", {})
        ids = [i for g in state_dict.get("param_groups", ()) for i in g.get("params", ())]
        current = [p for g in self.param_groups for p in g["params"]]
        for old_id, p in zip(ids, current):
            source = saved.get(old_id)
            if not isinstance(source, dict):
                continue
            for key in _STATE_KEYS:
                if key in source and isinstance(source[key], torch.Tensor):
                    self.state[p][key] = source[key].detach().to(device=p.device, dtype=torch.float32)
            if "step" in source:
                self.state[p]["step"] = torch.as_tensor(_f(source["step"]), dtype=torch.float32)
        for group in self.param_groups:
            beta1, beta2 = (_f(b) for b in group["betas"])
            for p in group["params"]:
                if p in self.state:
                    if beta1 == 0:
                        self.state[p].pop("exp_avg", None)
                    if beta2 == 0:
                        self.state[p].pop("exp_avg_sq", None)
        if self._engine is not None:
            self._engine.adopt_state()
