"""Capture and exact restore of every random stream of a job.

A checkpoint stores, per rank, the Python and NumPy generator states (pickled, as uint8
tensors with their lengths), the torch CPU state and one CUDA generator state per visible
device, under ``ranks.rank_%08d``.  Restore is only defined for the same world size.  The
pickled blobs are read back with an unpickler that admits nothing but NumPy's array
reconstruction helpers, and every state is first tried on a private generator, so a bad
checkpoint cannot leave the process-global streams half restored.

Parity: reference ``wm/infra/rng_state.py:16-231`` (format ``wm-trainer-rng-v1``).
"""

from __future__ import annotations

import io
import pickle
import random
from collections.abc import Iterator, Mapping, Sequence
from contextlib import contextmanager
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

__all__ = [
    "RNG_CHECKPOINT_FORMAT",
    "capture_distributed_rng_state",
    "isolated_rng",
    "restore_distributed_rng_state",
    "validate_distributed_rng_state",
]

RNG_CHECKPOINT_FORMAT = "wm-trainer-rng-v1"
RNG_CHECKPOINT_SCHEMA_VERSION = 1

_ALLOWED_GLOBALS = frozenset({
    ("numpy", "dtype"), ("numpy", "ndarray"),
    ("numpy._core.multiarray", "_reconstruct"), ("numpy._core.numeric", "_frombuffer"),
    ("numpy.core.multiarray", "_reconstruct"), ("numpy.core.numeric", "_frombuffer"),
})


@contextmanager
def isolated_rng(*, cuda_devices: Sequence[int] | None = None) -> Iterator[None]:
    """Run a block without disturbing the Python, NumPy, torch CPU and CUDA streams."""
    py, npy = random.getstate(), np.random.get_state()
    if cuda_devices is not None:
        devices = list(cuda_devices)
    elif torch.cuda.is_available() and torch.cuda.is_initialized():
        devices = list(range(torch.cuda.device_count()))
    else:
        devices = []
    try:
        with torch.random.fork_rng(devices=devices):
            yield
    finally:
        random.setstate(py)
        np.random.set_state(npy)


def _where() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _key(rank: int) -> str:
    return f"rank_{rank:08d}"


def _blob(obj: Any) -> tuple[torch.Tensor, int]:
    payload = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    return torch.frombuffer(bytearray(payload), dtype=torch.uint8).clone(), len(payload)


class _Restricted(pickle.Unpickler):
    def find_class(self, module: str, name: str) -> Any:
        if (module, name) not in _ALLOWED_GLOBALS:
            raise pickle.UnpicklingError(f"RNG state may not reference {module}.{name}")
        return super().find_class(module, name)


def _unblob(value: Any, length: int, what: str) -> Any:
    if not torch.is_tensor(value):
        raise RuntimeError("RNG checkpoint contains a non-tensor serialized state")
    if value.device.type != "cpu" or value.dtype != torch.uint8 or value.ndim != 1:
        raise RuntimeError("RNG serialized state must be a one-dimensional CPU uint8 tensor, "
                           f"got device={value.device}, dtype={value.dtype}, shape={tuple(value.shape)}")
    if not 0 < length <= value.numel():
        raise RuntimeError("RNG checkpoint serialized state length is invalid")
    try:
        return _Restricted(io.BytesIO(value.contiguous().numpy().tobytes()[:length])).load()
    except (pickle.UnpicklingError, EOFError) as error:
        raise RuntimeError(f"RNG checkpoint {what} serialized state is invalid") from error


def _local(rank: int) -> dict[str, Any]:
    py_blob, py_len = _blob(random.getstate())
    np_blob, np_len = _blob(np.random.get_state())
    cuda = bool(torch.cuda.is_available() and torch.cuda.is_initialized())
    states = [s.cpu().clone() for s in torch.cuda.get_rng_state_all()] if cuda else []
    return {
        "global_rank": int(rank),
        "python_blob": py_blob, "python_length": py_len,
        "numpy_blob": np_blob, "numpy_length": np_len,
        "torch_cpu": torch.get_rng_state().cpu().clone(),
        "cuda_initialized": cuda,
        "cuda_device_count": len(states),
        "current_cuda_device": torch.cuda.current_device() if cuda else -1,
        "cuda_states": {f"device_{i:04d}": s for i, s in enumerate(states)},
    }


def capture_distributed_rng_state() -> dict[str, Any]:
    rank, world = _where()
    mine = _local(rank)
    if world > 1:
        everyone: list[Any] = [None] * world
        dist.all_gather_object(everyone, mine)
        states = [s for s in everyone if s is not None]
    else:
        states = [mine]
    return {"format": RNG_CHECKPOINT_FORMAT, "schema_version": RNG_CHECKPOINT_SCHEMA_VERSION,
            "world_size": world, "ranks": {_key(i): s for i, s in enumerate(states)}}


def _decode(state: Mapping[str, Any]):
    if state.get("format") != RNG_CHECKPOINT_FORMAT or \
            state.get("schema_version") != RNG_CHECKPOINT_SCHEMA_VERSION:
        raise RuntimeError("Unsupported WM trainer RNG checkpoint format")
    rank, world = _where()
    if int(state.get("world_size", -1)) != world:
        raise RuntimeError(f"RNG checkpoint world-size mismatch: "
                           f"checkpoint={state.get('world_size')}, current={world}")
    ranks = state.get("ranks")
    if not isinstance(ranks, Mapping) or set(ranks) != {_key(i) for i in range(world)}:
        raise RuntimeError("RNG checkpoint rank topology does not match the current process group")
    item = ranks[_key(rank)]
    if not isinstance(item, Mapping):
        raise RuntimeError("RNG checkpoint rank entry is not a mapping")
    if item.get("global_rank") != rank:
        raise RuntimeError("RNG checkpoint rank entry belongs to a different rank")
    py = _unblob(item["python_blob"], int(item["python_length"]), "Python")
    npy = _unblob(item["numpy_blob"], int(item["numpy_length"]), "NumPy")
    cpu = item["torch_cpu"]
    if not torch.is_tensor(cpu):
        raise RuntimeError("RNG checkpoint contains a non-tensor serialized state")
    # dry run on private generators before any global stream is touched
    random.Random(0).setstate(py)
    np.random.RandomState(0).set_state(npy)
    torch.Generator(device="cpu").set_state(cpu)
    cuda_states = item.get("cuda_states", {})  # an empty mapping is not stored by DCP
    if not isinstance(cuda_states, Mapping):
        raise RuntimeError("RNG checkpoint CUDA state is not a mapping")
    ordered: list[torch.Tensor] = []
    if bool(item["cuda_initialized"]):
        if not torch.cuda.is_available():
            raise RuntimeError("RNG checkpoint contains CUDA state but CUDA is unavailable")
        count = torch.cuda.device_count()
        if int(item["cuda_device_count"]) != count:
            raise RuntimeError("RNG checkpoint CUDA device count differs")
        names = [f"device_{i:04d}" for i in range(count)]
        if set(cuda_states) != set(names):
            raise RuntimeError("RNG checkpoint CUDA device entries differ")
        ordered = [cuda_states[n] for n in names]
        for index, s in enumerate(ordered):
            torch.Generator(device=torch.device("cuda", index)).set_state(s)
    return py, npy, cpu, ordered


def validate_distributed_rng_state(state: Mapping[str, Any]) -> None:
    _decode(state)


def restore_distributed_rng_state(state: Mapping[str, Any]) -> None:
    py, npy, cpu, cuda = _decode(state)
    if cuda:
        torch.cuda.set_rng_state_all(cuda)
    torch.set_rng_state(cpu)
    np.random.set_state(npy)
    random.setstate(py)
