"""Flat tensor files (the ``.safetensors`` layout) read and written without a dependency.

Layout: an 8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end)}`` relative to the end of the header,
then the raw little-endian bytes.

Loading is a three-stage pipeline sized for a large-memory GPU node: (1) a native thread
pool issues positional reads of many tensors at once into a pinned slab, (2) each tensor
is copied (and converted) into its parameter with an asynchronous host-to-device copy on
a side stream, (3) the next slab is being read while the previous one is in flight; a slab
is reused only after the event recorded behind its last copy has completed.

Parity: reference ``wm/inference/cosmos3.py:241-304`` (parallel ``preadv`` of a tensor file
into parameters, largest tensors first, shape validation).
"""

from __future__ import annotations

import json
import os
import struct
from collections.abc import Iterable, Mapping
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Any

import torch

__all__ = ["DTYPES", "copy_into", "read_header", "read_tensors", "write_tensors"]

DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
          "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
          "U8": torch.uint8, "BOOL": torch.bool}
_NAMES = {dtype: name for name, dtype in DTYPES.items()}
READ_THREADS = 16
READ_CHUNK = 64 << 20
SLAB_BYTES = 512 << 20
_ALIGN = 64


def _native():
    try:
        from agentgarten_b200 import _io
        return _io
    except ImportError:
        return None


def read_header(path: str | Path) -> tuple[int, dict[str, dict[str, Any]], dict[str, str]]:
    """``(data_start, entries, metadata)`` of a tensor file."""
    with open(path, "rb") as handle:
        raw = handle.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path} is not a tensor file")
        (length,) = struct.unpack("<Q", raw)
        entries = json.loads(handle.read(length))
    metadata = entries.pop("__metadata__", None) or {}
    return 8 + length, entries, metadata


def write_tensors(tensors: Mapping[str, torch.Tensor], path: str | Path,
                  metadata: Mapping[str, str] | None = None) -> None:
    """Write ``tensors`` in name order; atomic through a temporary file beside the target."""
    header: dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    cursor = 0
    order = sorted(tensors)
    for name in order:
        value = tensors[name]
        if value.dtype not in _NAMES:
            raise TypeError(f"dtype {value.dtype} of {name!r} has no tensor-file code")
        size = value.numel() * value.element_size()
        header[name] = {"dtype": _NAMES[value.dtype], "shape": list(value.shape),
                        "data_offsets": [cursor, cursor + size]}
        cursor += size
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(8 + len(blob)) % 8)  # keep the data 8-byte aligned
    target = Path(path)
    scratch = target.with_name(target.name + f".tmp{os.getpid()}")
    with open(scratch, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in order:
            value = tensors[name].detach().contiguous().cpu()
            handle.write(value.view(torch.uint8).numpy().tobytes() if value.numel() else b"")
        handle.flush()
        os.fsync(handle.fileno())
    os.replace(scratch, target)


def _read_into(path: str, ranges: list[tuple[int, int, int]], views: list[memoryview | None]) -> None:
    native = _native()
    if native is not None:
        native.read_ranges(path, ranges, READ_THREADS, READ_CHUNK)
        return
    fd = os.open(path, os.O_RDONLY)  # interpreter fallback: same scheme with a Python pool
    try:
        def one(job):
            (offset, size, _), view = job
            done = 0
            while done < size:
                got = os.preadv(fd, [view[done:done + READ_CHUNK]], offset + done)
                if got <= 0:
                    raise OSError(f"truncated read at {offset + done} in {path}")
                done += got
        with ThreadPoolExecutor(READ_THREADS) as pool:
            list(pool.map(one, zip(ranges, views)))
    finally:
        os.close(fd)


def copy_into(path: str | Path, destinations: Mapping[str, torch.Tensor],
              keys: Mapping[str, str] | None = None, *, slab_bytes: int = SLAB_BYTES) -> set[str]:
    """Fill ``destinations[name]`` from file entry ``keys[name]`` (default: the same name).

    Shapes must match; dtypes are converted by the copy. Returns the destination names.
    """
    path = str(path)
    data_start, entries, _ = read_header(path)
    keys = dict(keys) if keys is not None else {name: name for name in destinations}
    jobs = []
    for name, key in keys.items():
        entry = entries[key]
        if tuple(entry["shape"]) != tuple(destinations[name].shape):
            raise ValueError(f"shape mismatch for {key!r} in {path}: file {tuple(entry['shape'])}, "
                             f"model {tuple(destinations[name].shape)}")
        begin, end = entry["data_offsets"]
        jobs.append((begin, end - begin, name, entry))
    if not jobs:
        return set()
    jobs.sort()  # file order: neighbouring reads, and slabs that fill evenly
    on_gpu = any(t.is_cuda for t in destinations.values())
    largest = max(size for _, size, _, _ in jobs)
    capacity = max(slab_bytes, largest + _ALIGN)
    slabs = [torch.empty(capacity, dtype=torch.uint8, pin_memory=on_gpu) for _ in range(2 if on_gpu else 1)]
    events: list[Any] = [None] * len(slabs)
    stream = torch.cuda.Stream() if on_gpu else None
    batch: list[tuple[int, int, str, dict, int]] = []
    turn = 0

    def flush() -> None:
        nonlocal batch, turn
        if not batch:
            return
        slab = slabs[turn % len(slabs)]
        if events[turn % len(slabs)] is not None:
            events[turn % len(slabs)].synchronize()
        base = slab.data_ptr()
        whole = memoryview(slab.numpy()) if _native() is None else None
        ranges = [(data_start + begin, size, base + at) for begin, size, _, _, at in batch]
        views = [None if whole is None else whole[at:at + size] for _, size, _, _, at in batch]
        _read_into(path, ranges, views)
        with torch.no_grad():
            for _, size, name, entry, at in batch:
                source = slab[at:at + size].view(DTYPES[entry["dtype"]]).view(entry["shape"])
                if stream is not None:
                    with torch.cuda.stream(stream):
                        destinations[name].copy_(source, non_blocking=True)
                else:
                    destinations[name].copy_(source)
        if stream is not None:
            events[turn % len(slabs)] = stream.record_event()
        batch = []
        turn += 1

    cursor = 0
    for begin, size, name, entry in jobs:
        if cursor + size > capacity:
            flush()
            cursor = 0
        batch.append((begin, size, name, entry, cursor))
        cursor += -(-size // _ALIGN) * _ALIGN
    flush()
    if stream is not None:
        stream.synchronize()
    return set(keys)


def read_tensors(path: str | Path, names: Iterable[str] | None = None,
                 device: str | torch.device = "cpu") -> dict[str, torch.Tensor]:
    """Materialise (a subset of) a tensor file as new tensors on ``device``."""
    _, entries, _ = read_header(path)
    wanted = list(entries) if names is None else list(names)
    out = {name: torch.empty(entries[name]["shape"], dtype=DTYPES[entries[name]["dtype"]], device=device)
           for name in wanted}
    copy_into(path, out)
    return out
