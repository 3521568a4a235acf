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
    horizon = config["dataloader_val"]["dataset"]["num_frames"]
    valid = type(horizon) is int and horizon > 1 and horizon % 4 == 1
    if not valid:
        raise ValueError(f"caption horizon must be 1 + 4N pixel frames, got {horizon!r}")
    return horizon


class _Run:
    """What a run's resolved ``config.yaml`` (a plain YAML tree, nothing is instantiated) says
    about the served towers.  Relative paths in it are relative to ``base``."""

    def __init__(self, tree: Mapping[str, Any], base: Path) -> None:
        self.tree, self.base = tree, base
        model = tree["model"]
        self.role = "student" if "student" in model else "net"   # distilled runs serve the student
        self.node = model[self.role]
        shape = self.node["config"]
        if not isinstance(shape, Mapping):
            raise ValueError(f"unresolved network config: {shape!r}")
        accepted = {field.name for field in fields(Cosmos3Config)}
        self.config = Cosmos3Config(**{key: shape[key] for key in shape if key in accepted})

    def path(self, text: str) -> Path:
        location = Path(text).expanduser()
        return (location if location.is_absolute() else self.base / location).resolve()

    @property
    def tokenizer(self) -> Path:
        return self.path(self.tree["model"]["conditioner"]["tokenizer_path"])

    def initial_weights(self) -> tuple[list[WeightSource], list[WeightSource]]:
        """The run's ``train.model_initializations`` sorted into (served tower, text tower)."""
        served: list[WeightSource] = []
        text: list[WeightSource] = []
        for overlay in (self.tree["train"].get("model_initializations") or {}).values():
            if overlay.get("path") is None:
                continue
            source = WeightSource(
                self.path(overlay["path"]),
                (overlay.get("source_model_key_prefix") or "").removeprefix("model."),
                tuple(overlay.get("source_model_key_patterns") or ()))
            targets = overlay.get("model_key_prefixes") or (overlay.get("model_key_prefix"),)
            if self.role in targets:
                served.append(source)
            if _TEXT_PREFIX in targets:
                text.append(source)
        return served, text

    def spec(self, checkpoint: Path, served, text, iteration: int) -> Cosmos3ArtifactSpec:
        return Cosmos3ArtifactSpec(checkpoint=checkpoint, config=self.config, student=tuple(served),
                                   text=tuple(text), tokenizer_path=self.tokenizer,
                                   prompt_pixel_frames=prompt_pixel_frames(self.tree),
                                   iteration=iteration, lora=self.node.get("lora"))


def _config_beside(checkpoint: Path) -> Path:
    """``config.yaml`` of the run: in the checkpoint, in the job directory two levels up
    (``job/checkpoints/iter_N``), or next to the checkpoint."""
    for folder in (checkpoint, checkpoint.parent.parent, checkpoint.parent):
        if (folder / "config.yaml").is_file():
            return folder / "config.yaml"
    raise FileNotFoundError(f"no resolved config.yaml beside {checkpoint}")


def inspect_artifact(checkpoint: str | Path) -> Cosmos3ArtifactSpec:
    checkpoint = Path(checkpoint).expanduser().resolve()
    folder = checkpoint.parent if checkpoint.is_file() else checkpoint
    if (folder / "manifest.json").is_file():
        return _inspect_export(folder)
    if not (checkpoint / "tensor" / ".metadata").is_file():
        raise FileNotFoundError(f"expected a DCP checkpoint with tensor/.metadata: {checkpoint}")
    config_path = _config_beside(checkpoint)
    run = _Run(yaml.safe_load(config_path.read_text()), config_path.parent)
    served, text = run.initial_weights()
    from torch.distributed.checkpoint import FileSystemReader

    stored = FileSystemReader(str(checkpoint / "tensor")).read_metadata().state_dict_metadata
    if f"model.{_TEXT_PREFIX}.embed_tokens.weight" in stored:   # the run saved its text tower too
        text.append(WeightSource(checkpoint, _TEXT_PREFIX))
    if not text:
        raise ValueError("checkpoint does not identify its frozen UND weight source")
    served.append(WeightSource(checkpoint, run.role))  # last: the checkpoint overlays what it owns
    number = re.fullmatch(r"iter_(\d+)", checkpoint.name)
    return run.spec(checkpoint, served, text, int(number.group(1)) if number else 0)


def _inspect_export(root: Path) -> Cosmos3ArtifactSpec:
    manifest = json.loads((root / "manifest.json").read_text())
    if (manifest.get("schema"), manifest.get("version")) != (MANIFEST_SCHEMA, MANIFEST_VERSION):
        raise ValueError("unsupported serving manifest schema/version")

    def local_file(name: str) -> Path:
        candidate = (root / name).resolve()
        if candidate.is_file() and candidate.is_relative_to(root):
            return candidate
        raise ValueError(f"serving manifest must name an existing local file: {name!r}")

    run = _Run(yaml.safe_load(local_file(manifest.get("config", "config.yaml")).read_text()), root)
    iteration = manifest["iteration"]
    if type(iteration) is not int or iteration < 0:
        raise ValueError("manifest iteration must be a nonnegative integer")
    # exported tensors carry module-local names, hence the empty prefixes
    towers = {role: (WeightSource(local_file(manifest[role]["file"]), ""),) for role in ("student", "und")}
    return run.spec(root, towers["student"], towers["und"], iteration)


def _refuse_stray_lora(names: Iterable[str]) -> None:
    """Adapter tensors that no ``lora`` declaration accounts for would be dropped silently."""
    stray = sorted(name for name in names if ".lora_" in name)
    if stray:
        raise ValueError(f"checkpoint has undeclared LoRA weights: {stray[:4]}")


class _TowerLoader:
    """Fills one materialised tower from its overlays, in order, and checks full coverage."""

    def __init__(self, tower: nn.Module, sources: tuple[WeightSource, ...]) -> None:
        self.tower, self.sources = tower, sources
        self.filled: set[str] = set()

    def _from_tensor_file(self, source: WeightSource) -> None:
        lead = source.prefix.rstrip(".") + "." if source.prefix else ""
        live = dict(self.tower.named_parameters())
        _, stored, _ = tensor_file.read_header(source.path)
        wanted = {name: lead + name for name in live if lead + name in stored}
        unused = stored.keys() - set(wanted.values())
        _refuse_stray_lora(name for name in unused if name.startswith(lead))
        with torch.no_grad():
            self.filled |= tensor_file.copy_into(source.path, {name: live[name] for name in wanted}, wanted)

    def _from_checkpoint(self, source: WeightSource) -> None:
        from agentgarten_b200.infra.checkpoint import DistributedCheckpointer

        outcome = DistributedCheckpointer(source.path.parent).load(
            self.tower, path=source.path, components=("model",), model_key_prefix="",
            source_model_key_prefix=source.prefix, source_model_key_patterns=source.patterns)
        _refuse_stray_lora(outcome.unexpected_model_keys)
        self.filled |= set(outcome.loaded_model_keys)

    def run(self) -> None:
        for source in self.sources:
            if source.path.suffix == ".safetensors":
                self._from_tensor_file(source)
            else:
                self._from_checkpoint(source)
        missing = sorted(set(self.tower.state_dict()) - self.filled)
        if missing:
            raise ValueError(f"inference weights are incomplete: {missing[:12]}")


def load_artifact(spec: Cosmos3ArtifactSpec, *, device: str | torch.device = "cuda",
                  dtype: torch.dtype = torch.bfloat16,
                  progress: Callable[[str, int, int], None] | None = None) -> Cosmos3Artifact:
    """Materialise the student and the text tower (with declared LoRA) and nothing else."""
    report = progress if progress is not None else (lambda *_: None)
    served = build_network(spec.config, init_device="meta", lora=dict(spec.lora) if spec.lora else None)
    with torch.device("meta"):
        text = Cosmos3TextEncoder(spec.config)
    for label, tower, sources in (("und", text, spec.text), ("student", served, spec.student)):
        report(label, 0, 0)
        tower.to(dtype=dtype).to_empty(device=device)
        _TowerLoader(tower, sources).run()
        tower.eval().requires_grad_(False)
        total = len(tower.state_dict())
        report(label, total, total)
    return Cosmos3Artifact(served, text, spec)


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
