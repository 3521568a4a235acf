"""Trained towers for inference: inspect a run, load only what serving needs, export it.

Two kinds of input are understood. A *training checkpoint* (``.../checkpoints/iter_N`` with
``tensor/.metadata``) is described by the resolved ``config.yaml`` of its run: the student
(or ``net``) tower is the run's initial weights overlaid by the checkpoint, the text tower
comes from the run's frozen source. An *export* (a directory with ``manifest.json``) holds
one flat tensor file per tower. Inspection only reads metadata: no recipe is imported and
no configuration target is executed. Loading builds the two towers on the meta device,
gives them storage on the target device and streams the tensors in (pipelined positional
reads for tensor files, the training restore path for sharded checkpoints); every live
parameter must be covered, and LoRA tensors nobody declared are an error.

Parity: reference ``wm/inference/cosmos3.py:54-403``.
"""

from __future__ import annotations

import json
import re
from collections.abc import Callable, Iterable, Mapping
from dataclasses import asdict, dataclass, fields
from pathlib import Path
from typing import Any

import torch
import yaml
from torch import nn

from agentgarten_b200.inference import tensor_file
from agentgarten_b200.networks.cosmos3 import (Cosmos3Config, Cosmos3Network, Cosmos3TextEncoder,
                                               build_network)

__all__ = ["Cosmos3Artifact", "Cosmos3ArtifactSpec", "WeightSource", "inspect_artifact",
           "load_artifact", "prompt_pixel_frames", "save_artifact"]

MANIFEST_SCHEMA = "v2v.raw-dmd-safetensors"
MANIFEST_VERSION = 1
_TEXT_PREFIX = "conditioner.text_encoder"


@dataclass(frozen=True, slots=True)
class WeightSource:
    """One overlay: where tensors come from, under which prefix, and which of them."""

    path: Path
    prefix: str
    patterns: tuple[str, ...] = ()


@dataclass(frozen=True, slots=True)
class Cosmos3ArtifactSpec:
    """Everything needed to load, resolved to absolute paths."""

    checkpoint: Path
    config: Cosmos3Config
    student: tuple[WeightSource, ...]
    text: tuple[WeightSource, ...]
    tokenizer_path: Path
    prompt_pixel_frames: int
    iteration: int
    lora: Mapping[str, Any] | None = None  # keyword arguments of ``networks.lora.inject_lora``


@dataclass
class Cosmos3Artifact:
    """Resident generation and text towers; per-session stream state lives elsewhere."""

    student: Cosmos3Network
    context_encoder: Cosmos3TextEncoder
    spec: Cosmos3ArtifactSpec

    @property
    def tokenizer_path(self) -> Path:
        return self.spec.tokenizer_path

    @property
    def prompt_pixel_frames(self) -> int:
        return self.spec.prompt_pixel_frames

    @property
    def special_tokens(self) -> dict[str, int]:
        return self.spec.config.special_tokens

    @property
    def report(self) -> dict[str, object]:
        """Small JSON-compatible provenance for a status panel."""
        return {
            "implementation": "agentgarten_b200.networks.cosmos3",
            "checkpoint_path": str(self.spec.checkpoint),
            "iteration": self.spec.iteration,
            "und_checkpoint_path": str(self.spec.text[-1].path),
            "lora_loaded": self.spec.lora is not None,
            "first_frame_reference_embedding": self.spec.config.first_frame_reference_embedding,
        }


def prompt_pixel_frames(config: Mapping[str, Any]) -> int:
    """The caption horizon (pixel frames) the run was trained with: ``1 + 4N``."""
    count = config["dataloader_val"]["dataset"]["num_frames"]
    if type(count) is not int or count <= 1 or (count - 1) % 4:
        raise ValueError(f"caption horizon must be 1 + 4N pixel frames, got {count!r}")
    return count


def _absolute(path: str, root: Path) -> Path:
    location = Path(path).expanduser()
    return (location if location.is_absolute() else root / location).resolve()


def _tower(config: Mapping[str, Any]) -> tuple[str, Mapping[str, Any], Cosmos3Config]:
    """Which model entry owns the served weights (``student`` when distilled, else ``net``)."""
    model = config["model"]
    role = "student" if "student" in model else "net"
    node = model[role]
    raw = node["config"]
    if not isinstance(raw, Mapping):
        raise ValueError(f"unresolved network config: {raw!r}")
    known = {f.name for f in fields(Cosmos3Config)}
    return role, node, Cosmos3Config(**{k: v for k, v in raw.items() if k in known})


def inspect_artifact(checkpoint: str | Path) -> Cosmos3ArtifactSpec:
    checkpoint = Path(checkpoint).expanduser().resolve()
    holder = checkpoint.parent if checkpoint.is_file() else checkpoint
    if (holder / "manifest.json").is_file():
        return _inspect_export(holder)
    if not (checkpoint / "tensor" / ".metadata").is_file():
        raise FileNotFoundError(f"expected a DCP checkpoint with tensor/.metadata: {checkpoint}")
    places = (checkpoint / "config.yaml", checkpoint.parent.parent / "config.yaml",
              checkpoint.parent / "config.yaml")
    config_path = next((p for p in places if p.is_file()), None)
    if config_path is None:
        raise FileNotFoundError(f"no resolved config.yaml beside {checkpoint}")
    config = yaml.safe_load(config_path.read_text())
    role, node, topology = _tower(config)

    student: list[WeightSource] = []
    text: list[WeightSource] = []
    for entry in (config["train"].get("model_initializations") or {}).values():
        if entry.get("path") is None:
            continue
        destinations = entry.get("model_key_prefixes") or (entry.get("model_key_prefix"),)
        source = WeightSource(_absolute(entry["path"], config_path.parent),
                              (entry.get("source_model_key_prefix") or "").removeprefix("model."),
                              tuple(entry.get("source_model_key_patterns") or ()))
        if role in destinations:
            student.append(source)
        if _TEXT_PREFIX in destinations:
            text.append(source)
    from torch.distributed.checkpoint import FileSystemReader

    saved = FileSystemReader(str(checkpoint / "tensor")).read_metadata().state_dict_metadata
    if f"model.{_TEXT_PREFIX}.embed_tokens.weight" in saved:
        text.append(WeightSource(checkpoint, _TEXT_PREFIX))
    if not text:
        raise ValueError("checkpoint does not identify its frozen UND weight source")
    student.append(WeightSource(checkpoint, role))  # the checkpoint overlays what it owns
    numbered = re.fullmatch(r"iter_(\d+)", checkpoint.name)
    return Cosmos3ArtifactSpec(
        checkpoint=checkpoint, config=topology, student=tuple(student), text=tuple(text),
        tokenizer_path=_absolute(config["model"]["conditioner"]["tokenizer_path"], config_path.parent),
        prompt_pixel_frames=prompt_pixel_frames(config),
        iteration=int(numbered[1]) if numbered else 0, lora=node.get("lora"))


def _inspect_export(root: Path) -> Cosmos3ArtifactSpec:
    manifest = json.loads((root / "manifest.json").read_text())
    if manifest.get("schema") != MANIFEST_SCHEMA or manifest.get("version") != MANIFEST_VERSION:
        raise ValueError("unsupported serving manifest schema/version")

    def inside(name: str) -> Path:
        path = (root / name).resolve()
        if not path.is_relative_to(root) or not path.is_file():
            raise ValueError(f"serving manifest must name an existing local file: {name!r}")
        return path

    config = yaml.safe_load(inside(manifest.get("config", "config.yaml")).read_text())
    _, node, topology = _tower(config)
    iteration = manifest["iteration"]
    if type(iteration) is not int or iteration < 0:
        raise ValueError("manifest iteration must be a nonnegative integer")
    # exported tensors carry module-local names: no prefix
    student, text = (WeightSource(inside(manifest[role]["file"]), "") for role in ("student", "und"))
    return Cosmos3ArtifactSpec(
        checkpoint=root, config=topology, student=(student,), text=(text,),
        tokenizer_path=_absolute(config["model"]["conditioner"]["tokenizer_path"], root),
        prompt_pixel_frames=prompt_pixel_frames(config), iteration=iteration, lora=node.get("lora"))


def _reject_undeclared_lora(keys: Iterable[str]) -> None:
    stray = sorted(k for k in keys if ".lora_" in k)
    if stray:
        raise ValueError(f"checkpoint has undeclared LoRA weights: {stray[:4]}")


def _load_tensor_file(module: nn.Module, source: WeightSource) -> set[str]:
    prefix = source.prefix.rstrip(".") + "." if source.prefix else ""
    parameters = dict(module.named_parameters())
    _, entries, _ = tensor_file.read_header(source.path)
    chosen = {name: prefix + name for name in parameters if prefix + name in entries}
    _reject_undeclared_lora(k for k in entries.keys() - set(chosen.values()) if k.startswith(prefix))
    with torch.no_grad():
        return tensor_file.copy_into(source.path, {n: parameters[n] for n in chosen}, chosen)


def _load_tower(module: nn.Module, sources: tuple[WeightSource, ...]) -> None:
    from agentgarten_b200.infra.checkpoint import DistributedCheckpointer

    restorer = DistributedCheckpointer(sources[-1].path.parent)
    covered: set[str] = set()
    for source in sources:
        if source.path.suffix == ".safetensors":
            covered |= _load_tensor_file(module, source)
            continue
        result = restorer.load(module, path=source.path, components=("model",),
                               source_model_key_prefix=source.prefix, model_key_prefix="",
                               source_model_key_patterns=source.patterns)
        _reject_undeclared_lora(result.unexpected_model_keys)
        covered |= set(result.loaded_model_keys)
    absent = set(module.state_dict()) - covered
    if absent:
        raise ValueError(f"inference weights are incomplete: {sorted(absent)[:12]}")


def load_artifact(spec: Cosmos3ArtifactSpec, *, device: str | torch.device = "cuda",
                  dtype: torch.dtype = torch.bfloat16,
                  progress: Callable[[str, int, int], None] | None = None) -> Cosmos3Artifact:
    """Materialise the student and the text tower (with declared LoRA) and nothing else."""
    student = build_network(spec.config, init_device="meta", lora=dict(spec.lora) if spec.lora else None)
    with torch.device("meta"):
        text = Cosmos3TextEncoder(spec.config)
    for label, tower, sources in (("und", text, spec.text), ("student", student, spec.student)):
        if progress is not None:
            progress(label, 0, 0)
        tower.to(dtype=dtype).to_empty(device=device)
        _load_tower(tower, sources)
        tower.eval().requires_grad_(False)
        if progress is not None:
            count = len(tower.state_dict())
            progress(label, count, count)
    return Cosmos3Artifact(student, text, spec)


def _plain(value: Any) -> Any:
    if isinstance(value, Mapping):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    return value


def save_artifact(artifact: Cosmos3Artifact, directory: str | Path) -> Path:
    """Write both towers as flat tensor files plus the manifest :func:`inspect_artifact` reads."""
    root = Path(directory).expanduser().resolve()
    root.mkdir(parents=True, exist_ok=True)
    spec = artifact.spec
    manifest: dict[str, Any] = {"schema": MANIFEST_SCHEMA, "version": MANIFEST_VERSION,
                                "iteration": spec.iteration, "config": "config.yaml"}
    for role, tower in (("student", artifact.student), ("und", artifact.context_encoder)):
        name = f"{role}.safetensors"
        tensor_file.write_tensors({k: v.detach() for k, v in tower.state_dict().items()}, root / name,
                                  metadata={"format": "pt"})
        manifest[role] = {"file": name}
    config = {
        "model": {"student": {"config": _plain(asdict(spec.config)),
                              "lora": None if spec.lora is None else _plain(spec.lora)},
                  "conditioner": {"tokenizer_path": str(spec.tokenizer_path)}},
        "dataloader_val": {"dataset": {"num_frames": spec.prompt_pixel_frames}},
    }
    (root / "config.yaml").write_text(yaml.safe_dump(config))
    (root / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    return root
