"""Opening a checkpoint for reading, whatever its layout.

Accepted layouts: a training checkpoint (``<dir>/tensor/.metadata``), a bare DCP directory
(``<dir>/.metadata``), a DCP model directory (``<dir>/model/.metadata``) and a HuggingFace
safetensors directory.  HuggingFace directories and raw DCP overlays store model tensors at
the top level instead of under ``model.``.

Parity: reference ``wm/infra/checkpoint/source.py:29-125``.
"""

from __future__ import annotations

from collections.abc import Iterable
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .common import ALL_COMPONENTS, TENSOR_COMPONENTS

__all__ = ["LoadSource", "component_fields", "component_names", "normalise_components"]


def _reader_for(path: Path):
    from torch.distributed.checkpoint import FileSystemReader

    for candidate in (path / "tensor", path, path / "model"):
        if (candidate / ".metadata").is_file():
            return FileSystemReader(str(candidate)), False
    from torch.distributed.checkpoint import HuggingFaceStorageReader

    return HuggingFaceStorageReader(str(path)), True


def component_names(keys: Iterable[str], component: str) -> set[str]:
    """Second-level names below ``component.`` (e.g. optimizer roles)."""
    head = f"{component}."
    return {k[len(head):].split(".", 1)[0] for k in keys if k.startswith(head) and len(k) > len(head)}


def component_fields(keys: Iterable[str], component: str, name: str | None = None) -> set[str]:
    head = f"{component}." if name is None else f"{component}.{name}."
    return {k[len(head):] for k in keys if k.startswith(head) and len(k) > len(head)}


def normalise_components(components: Iterable[str] | None, *, include_dataloader: bool = False,
                         ) -> tuple[str, ...]:
    if components is None:
        return ALL_COMPONENTS if include_dataloader else TENSOR_COMPONENTS
    wanted = set(components)
    unknown = wanted - set(ALL_COMPONENTS)
    if unknown:
        raise ValueError(f"Unknown checkpoint components: {', '.join(sorted(unknown))}")
    return tuple(c for c in ALL_COMPONENTS if c in wanted)


@dataclass(frozen=True, slots=True)
class LoadSource:
    reader: Any
    metadata: Any
    state_keys: set[str]
    is_huggingface: bool
    flat_model: bool
    saved_components: frozenset[str]

    @classmethod
    def open(cls, checkpoint_path: Path, source_model_key_prefix: str | None) -> "LoadSource":
        reader, hf = _reader_for(Path(checkpoint_path))
        metadata = reader.read_metadata()
        keys = {str(k) for k in metadata.state_dict_metadata}
        nested = any(k.startswith("model.") for k in keys)
        raw_overlay = (not hf and source_model_key_prefix is not None and not nested and bool(keys))
        flat = hf or raw_overlay
        components = frozenset({"model"} if flat and keys else {k.split(".", 1)[0] for k in keys})
        return cls(reader, metadata, keys, hf, flat, components)

    def has(self, component: str, selected: Iterable[str]) -> bool:
        return component in selected and component in self.saved_components
