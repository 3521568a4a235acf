"""Host-side reading of the per-device kernel status word.

Every bounded wait of this package's CUDA kernels (mbarrier, peer counter, tensor-parallel
flag) that runs out records a code in one int32 word per device and makes the kernel return
without finishing its work; later waits then give up at once.  Nothing on the device can
stop the host from carrying on with the unfinished outputs, so the host has to look at the
word where it reads from the device anyway: the non-finite consensus of a training update,
before a checkpoint is written, and at the block boundary of a stream.  ``status_flag``
gives the word as an FP32 device scalar that can ride along an existing all-reduce(MAX);
``raise_for_status`` turns a non-zero value into :class:`KernelStatusError`.

A test (or a rank whose peer died) may set a host-side override with ``inject`` — the value
then stands in for the device word, which lets the multi-rank agreement be exercised on CPU
ranks without any GPU fault.
"""

from __future__ import annotations

import torch

__all__ = ["CODES", "KernelStatusError", "inject", "raise_for_status", "read", "status_flag"]

CODES = {
    1: "kTimeoutProducer (a TMA producer waited too long for a free stage)",
    2: "kTimeoutMma (the MMA issuer waited too long for a full stage or a free accumulator)",
    3: "kTimeoutEpilogue (an epilogue waited too long for an accumulator)",
    4: "kTimeoutSoftmax (a softmax warp waited too long)",
    5: "kTimeoutPeer (a flag owned by another GPU never arrived)",
    6: "kBadArgument (a work list does not fit the kernel's tables)",
    7: "kBadIndex (a work-list entry pointed outside its tensor; the CTA skipped its work)",
}

_injected: int | None = None


class KernelStatusError(RuntimeError):
    """A kernel of this package gave up on a bounded wait; its outputs are incomplete."""

    def __init__(self, code: int, where: str) -> None:
        self.code = int(code)
        name = CODES.get(self.code, f"code {self.code}")
        super().__init__(
            f"{where}: kernel status word = {self.code}: {name}.  A bounded wait ran out on at "
            "least one rank and the kernel returned early; tensors produced since then are "
            "incomplete and must not be trained on, served or checkpointed.")


def inject(code: int | None) -> None:
    """Host-side stand-in for the device word (``None`` removes it)."""
    global _injected
    _injected = None if code is None else int(code)


def status_flag(device: torch.device | str) -> torch.Tensor:
    """The status word of ``device`` as an FP32 scalar on that device (0 on the CPU or
    without the extension), without synchronising."""
    device = torch.device(device)
    if _injected is not None:
        return torch.tensor(float(_injected), device=device)
    if device.type != "cuda":
        return torch.zeros((), device=device)
    from agentgarten_b200.ops import native

    if not native.available():
        return torch.zeros((), device=device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    return native.ext().status(index).reshape(()).float()


def read(device: torch.device | str, group=None) -> int:
    """Status word, MAX over the ranks of ``group`` when a process group is up (one host read)."""
    import torch.distributed as dist

    flag = status_flag(device).clone()
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    return int(flag.item())


def raise_for_status(code: int | float, where: str) -> None:
    if int(code) != 0:
        raise KernelStatusError(int(code), where)
