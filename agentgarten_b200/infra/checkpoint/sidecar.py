"""Files beside the tensor checkpoint: job metadata and per-rank data-loader cursors.

``metadata.json``: ``{version, iteration, world_size, runtime}``.  ``dataloader/rank_%05d.pt``
holds each rank's loader cursor and ``dataloader/metadata.json`` the world size, mesh and
loader signature it belongs to.  A cursor is reused only when world size, mesh and
signature are identical; rank 0 decides and broadcasts, and any failure is raised on every
rank.

Parity: reference ``wm/infra/checkpoint/sidecar.py:19-352``.
"""

from __future__ import annotations

import io
import json
from collections.abc import Mapping
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist

from agentgarten_b200.utils.io import atomic_put, atomic_put_text

from .common import gather_objects, raise_together, rank, warn_rank0, world_size

__all__ = ["DataloaderSnapshot", "capture_dataloader_snapshot", "restore_dataloader_snapshot",
           "save_checkpoint_metadata", "save_dataloader_snapshot", "warn_runtime_metadata_changes"]

VERSION = 1


@dataclass
class DataloaderSnapshot:
    state: dict[str, Any] | None
    metadata: dict[str, Any]


def _plain(value: Any) -> Any:
    if isinstance(value, Mapping):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    if isinstance(value, (str, int, float, bool)) or value is None:
        return value
    return str(value)


def _signature(loader: Any) -> dict[str, Any]:
    describe = getattr(loader, "resume_signature", None)
    return {"num_workers": int(getattr(loader, "num_workers", 0) or 0),
            "loader": _plain(describe()) if callable(describe) else None}


def _stateful(loader: Any) -> bool:
    return loader is not None and callable(getattr(loader, "state_dict", None)) \
        and callable(getattr(loader, "load_state_dict", None))


def capture_dataloader_snapshot(dataloader: Any, runtime_metadata: Mapping[str, Any] | None = None,
                                ) -> DataloaderSnapshot | None:
    support = gather_objects(_stateful(dataloader))
    if not all(support):
        if any(support):
            warn_rank0("Only some ranks have a stateful dataloader; its cursor is not saved.")
        return None
    error, state = None, None
    try:
        state = dict(dataloader.state_dict())
    except BaseException as e:  # reported collectively below
        error = e
    raise_together("dataloader snapshot", error)
    return DataloaderSnapshot(state, {"version": VERSION, "world_size": world_size(),
                                      "mesh": _plain((runtime_metadata or {}).get("mesh")),
                                      "workers": _signature(dataloader)})


def save_dataloader_snapshot(checkpoint_path: str | Path, snapshot: DataloaderSnapshot | None) -> None:
    if snapshot is None:
        return
    checkpoint_path = Path(checkpoint_path)
    error = None
    try:
        buffer = io.BytesIO()
        torch.save(snapshot.state, buffer)
        atomic_put(buffer.getvalue(), checkpoint_path / "dataloader" / f"rank_{rank():05d}.pt")
        if rank() == 0:
            atomic_put_text(json.dumps(snapshot.metadata, sort_keys=True) + "\n",
                            checkpoint_path / "dataloader" / "metadata.json")
    except BaseException as e:
        error = e
    raise_together("dataloader sidecar write", error)


def save_checkpoint_metadata(checkpoint_path: str | Path, *, iteration: int,
                             runtime_metadata: Mapping[str, Any] | None = None) -> None:
    checkpoint_path = Path(checkpoint_path)
    error = None
    if rank() == 0:
        try:
            payload = {"version": VERSION, "iteration": int(iteration), "world_size": world_size(),
                       "runtime": _plain(dict(runtime_metadata or {}))}
            atomic_put_text(json.dumps(payload, sort_keys=True) + "\n", checkpoint_path / "metadata.json")
        except BaseException as e:
            error = e
    raise_together("metadata write", error)


def warn_runtime_metadata_changes(checkpoint_path: str | Path,
                                  runtime_metadata: Mapping[str, Any] | None = None) -> None:
    path = Path(checkpoint_path) / "metadata.json"
    if rank() != 0 or not path.is_file():
        return
    try:
        saved = json.loads(path.read_text())
    except (OSError, ValueError):
        return
    if int(saved.get("world_size", world_size())) != world_size():
        warn_rank0(f"Checkpoint was written by {saved.get('world_size')} ranks, resuming on "
                   f"{world_size()}: RNG streams and dataloader cursors are not restored.")
    now = _plain(dict(runtime_metadata or {}))
    if saved.get("runtime") not in (None, now) and now:
        warn_rank0("Runtime metadata (mesh / topology) differs from the checkpoint's.")


def restore_dataloader_snapshot(checkpoint_path: str | Path, dataloader: Any,
                                runtime_metadata: Mapping[str, Any] | None = None) -> bool:
    """Restore the cursor when the checkpoint's loader stream is the current one."""
    checkpoint_path = Path(checkpoint_path)
    support = gather_objects(_stateful(dataloader))
    if not all(support):
        return False
    decision: list[Any] = [False, None]
    if rank() == 0:
        meta_path = checkpoint_path / "dataloader" / "metadata.json"
        try:
            if meta_path.is_file():
                saved = json.loads(meta_path.read_text())
                same = (int(saved.get("world_size", -1)) == world_size()
                        and saved.get("mesh") == _plain((runtime_metadata or {}).get("mesh"))
                        and saved.get("workers") == _signature(dataloader))
                decision = [bool(same), None if same else "dataloader stream changed"]
            else:
                decision = [False, "no dataloader sidecar"]
        except (OSError, ValueError) as e:
            decision = [False, f"unreadable dataloader sidecar: {e}"]
    if world_size() > 1:
        dist.broadcast_object_list(decision, src=0)
    if not decision[0]:
        if decision[1] and decision[1] != "no dataloader sidecar":
            warn_rank0(f"Not restoring the dataloader cursor: {decision[1]}.")
        return False
    error = None
    try:
        state = torch.load(checkpoint_path / "dataloader" / f"rank_{rank():05d}.pt", weights_only=True)
        dataloader.load_state_dict(state)
    except BaseException as e:
        error = e
    raise_together("dataloader restore", error)
    return True
