"""Agreement across ranks on whether this update's gradients are finite.

Every active optimizer contributes a flag: the flat CUDA engine produces it as a side
output of its reduce-scatter kernel (already combined over the shard group); other
optimizers are scanned with a foreach finite check.  A GradScaler's own ``found_inf``
records are merged in.  The flags are combined with an all-reduce(MAX) and written back
into the GradScaler, so ``scaler.step``/``scaler.update`` take the same branch everywhere.
One device→host read per update.  The kernel status word of this rank's device travels in
the same all-reduce and the same read: a bounded wait that ran out in any kernel on any rank
(gradient exchange, context-parallel exchange, tensor-core pipelines) raises
``KernelStatusError`` here, before the optimizer consumes incomplete gradients.

Parity: reference ``wm/infra/nonfinite.py:20-119``.
"""

from __future__ import annotations

from collections import defaultdict

import torch
import torch.distributed as dist

from agentgarten_b200.ops.kernel_status import raise_for_status, status_flag

__all__ = ["synchronize_found_nonfinite"]


@torch.no_grad()
def _scan(optimizers) -> list[torch.Tensor]:
    flags: list[torch.Tensor] = []
    buckets: dict[tuple[torch.device, torch.dtype], list[torch.Tensor]] = defaultdict(list)
    seen: set[int] = set()
    for optimizer in optimizers:
        probe = getattr(optimizer, "found_nonfinite", None)
        flag = probe() if callable(probe) else None
        if flag is not None:
            flags.append(flag.reshape(()).float())
            continue
        for group in optimizer.param_groups:
            for p in group["params"]:
                if id(p) in seen or p.grad is None:
                    continue
                seen.add(id(p))
                grad = p.grad.to_local() if hasattr(p.grad, "to_local") else p.grad
                if grad.is_sparse:
                    grad = grad.coalesce().values()
                if grad.numel():
                    buckets[(grad.device, grad.dtype)].append(grad)
    per_device: dict[torch.device, torch.Tensor] = {}
    for (device, _dtype), grads in buckets.items():
        found = per_device.setdefault(device, torch.zeros((), dtype=torch.float32, device=device))
        worst = torch.stack([n.float() for n in torch._foreach_norm(grads, float("inf"))])
        found.copy_(torch.maximum(found, (~torch.isfinite(worst).all()).float()))
    flags.extend(per_device.values())
    return flags


def synchronize_found_nonfinite(grad_scaler, optimizers, *, fallback_device) -> bool:
    records = []
    flags: list[torch.Tensor] = []
    if grad_scaler is not None and grad_scaler.is_enabled():
        records = [grad_scaler._found_inf_per_device(opt) for opt in optimizers]
        flags = [flag for record in records for flag in record.values()]
    flags.extend(_scan(tuple(optimizers)))
    if flags:
        verdict = flags[0].detach().clone().float()
        for flag in flags[1:]:
            verdict.copy_(torch.maximum(verdict, flag.to(verdict.device).float()))
    else:
        verdict = torch.zeros((), dtype=torch.float32, device=fallback_device)
    verdict.clamp_(0, 1)
    word = torch.stack((verdict.reshape(()), status_flag(verdict.device).to(verdict.device)))
    if dist.is_available() and dist.is_initialized():
        # inside a node through the NVSwitch multicast mapping (one launch), else the library all-reduce
        from agentgarten_b200.parallel.consensus import maximum

        maximum(word)
    nonfinite, status = word.tolist()  # the one host read of the update
    raise_for_status(status, "training update")
    verdict = word[0].clamp_(0, 1)
    for record in records:
        if record:
            for device, flag in record.items():
                flag.copy_(verdict.to(device))
        else:
            record[verdict.device] = verdict.clone()
    return bool(nonfinite)
