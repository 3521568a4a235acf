"""Multi-tensor Adam entry points with Transformer Engine's signatures, on ``torch._fused_adamw_``.

``tensor_lists`` is ``[gradients, parameters, exp_avgs, exp_avg_sqs(, master_parameters)]``.
With master weights the FP32 masters are updated by the fused kernel from FP32 copies of the
gradients and the low-precision parameters are refreshed from them, which is what the
Transformer Engine kernel does in one pass.
"""

from __future__ import annotations

import torch


def _fused(gradients, targets, exp_avgs, exp_avg_sqs, *, lr, beta1, beta2, eps, step, adam_w_mode,
           bias_correction, weight_decay):
    if not bias_correction:
        raise NotImplementedError("the stand-in implements bias-corrected Adam only")
    device = targets[0].device
    step_tensor = step if isinstance(step, torch.Tensor) else torch.tensor(float(step), device=device)
    step_tensor = step_tensor.to(device=device, dtype=torch.float32).reshape(())
    steps = [step_tensor] * len(targets)
    work = [g if g.dtype == t.dtype else g.to(t.dtype) for g, t in zip(gradients, targets)]
    if isinstance(lr, torch.Tensor):
        lr = lr.to(device=device, dtype=torch.float32).reshape(())
    kernel = torch._fused_adamw_ if adam_w_mode else torch._fused_adam_
    kernel(list(targets), work, list(exp_avgs), list(exp_avg_sqs), [], steps, lr=lr, beta1=float(beta1),
           beta2=float(beta2), weight_decay=float(weight_decay), eps=float(eps), amsgrad=False,
           maximize=False, grad_scale=None, found_inf=None)


def multi_tensor_adam(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step, mode,
                      bias_correction, weight_decay):
    gradients, parameters, exp_avgs, exp_avg_sqs = tensor_lists
    _fused(gradients, parameters, exp_avgs, exp_avg_sqs, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
           step=step, adam_w_mode=bool(mode), bias_correction=bool(bias_correction),
           weight_decay=weight_decay)


def multi_tensor_adam_capturable(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step, mode,
                                 bias_correction, weight_decay, inv_scale):
    multi_tensor_adam(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step, mode,
                      bias_correction, weight_decay)


def multi_tensor_adam_capturable_master(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step,
                                        mode, bias_correction, weight_decay, inv_scale):
    gradients, parameters, exp_avgs, exp_avg_sqs, masters = tensor_lists
    _fused(gradients, masters, exp_avgs, exp_avg_sqs, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
           step=step, adam_w_mode=bool(mode), bias_correction=bool(bias_correction),
           weight_decay=weight_decay)
    torch._foreach_copy_(list(parameters), list(masters))
