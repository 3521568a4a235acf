"""Tensor files, the native parallel reader and the artifact inspect/load/export cycle."""

import pathlib

import pytest
import torch
import yaml

from agentgarten_b200.inference import tensor_file
from agentgarten_b200.inference.cosmos3 import (inspect_artifact, load_artifact, prompt_pixel_frames,
                                                save_artifact)
from agentgarten_b200.networks.cosmos3 import TEXT_ENCODER_KEYS, Cosmos3Config, Cosmos3TextEncoder

from test_train_cpu import _train


def _sample():
    torch.manual_seed(0)
    return {"a.weight": torch.randn(300, 70).bfloat16(), "b": torch.arange(10), "empty": torch.zeros(0, 3),
            "big": torch.randn(700, 1000), "flag": torch.tensor([True, False])}


def test_tensor_file_round_trip_and_interop(tmp_path):
    tensors = _sample()
    tensor_file.write_tensors(tensors, tmp_path / "own.safetensors", {"format": "pt"})
    start, entries, metadata = tensor_file.read_header(tmp_path / "own.safetensors")
    assert metadata == {"format": "pt"} and start % 8 == 0 and set(entries) == set(tensors)
    back = tensor_file.read_tensors(tmp_path / "own.safetensors")
    assert all(torch.equal(back[k], v) for k, v in tensors.items())
    safetensors = pytest.importorskip("safetensors.torch")
    theirs = safetensors.load_file(str(tmp_path / "own.safetensors"))
    assert all(torch.equal(theirs[k], v) for k, v in tensors.items())
    safetensors.save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "lib.safetensors"))
    back = tensor_file.read_tensors(tmp_path / "lib.safetensors", names=["big", "a.weight"])
    assert torch.equal(back["big"], tensors["big"]) and set(back) == {"big", "a.weight"}


def test_copy_into_converts_checks_shapes_and_survives_small_slabs(tmp_path, monkeypatch):
    tensors = _sample()
    tensor_file.write_tensors(tensors, tmp_path / "t.safetensors")
    for native in (True, False):
        if not native:
            monkeypatch.setattr(tensor_file, "_native", lambda: None)
        target = {"w": torch.zeros(300, 70), "x": torch.zeros(700, 1000)}
        done = tensor_file.copy_into(tmp_path / "t.safetensors", target, {"w": "a.weight", "x": "big"},
                                     slab_bytes=4096)
        assert done == {"w", "x"}
        assert torch.equal(target["w"], tensors["a.weight"].float()) and torch.equal(target["x"], tensors["big"])
    with pytest.raises(ValueError):
        tensor_file.copy_into(tmp_path / "t.safetensors", {"w": torch.zeros(3, 3)}, {"w": "a.weight"})


def test_native_reader_reports_truncation(tmp_path):
    _io = pytest.importorskip("agentgarten_b200._io")
    path = tmp_path / "blob.bin"
    path.write_bytes(bytes(range(200)))
    buffer = torch.zeros(200, dtype=torch.uint8)
    assert _io.read_ranges(str(path), [(0, 120, buffer.data_ptr()), (120, 80, buffer.data_ptr() + 120)], 4, 16) == 200
    assert buffer.tolist() == list(range(200)) and _io.file_size(str(path)) == 200
    with pytest.raises(RuntimeError):
        _io.read_ranges(str(path), [(150, 100, buffer.data_ptr())], 2, 16)
    with pytest.raises(RuntimeError):
        _io.read_ranges(str(tmp_path / "absent"), [(0, 1, buffer.data_ptr())], 2, 16)


def test_prompt_horizon_rule():
    assert prompt_pixel_frames({"dataloader_val": {"dataset": {"num_frames": 81}}}) == 81
    for bad in (80, 1, 5.0, True):
        with pytest.raises(ValueError):
            prompt_pixel_frames({"dataloader_val": {"dataset": {"num_frames": bad}}})


def test_artifact_from_a_training_run_and_from_its_export(tmp_path):
    run = tmp_path / "run"
    _train(["train.max_iterations=2", "train.checkpoint_interval=2", "train.validation_interval=100",
            "train.validate_at_start=false"], run)
    config = yaml.safe_load((run / "config.yaml").read_text())
    topology = {k: v for k, v in config["cosmos3"].items() if not k.startswith("_")}
    torch.manual_seed(3)
    text = Cosmos3TextEncoder(Cosmos3Config(**topology))
    released = run / "released" / "transformer"
    released.mkdir(parents=True)
    tensor_file.write_tensors(dict(text.state_dict()), released / "model.safetensors", {"format": "pt"})
    # what a released-weights recipe records about its frozen text tower and caption horizon
    config["model"]["conditioner"]["tokenizer_path"] = "released/text_tokenizer"
    config["dataloader_val"]["dataset"]["num_frames"] = 9
    config["train"]["model_initializations"] = {"text": {
        "path": "released/transformer", "model_key_prefix": "conditioner.text_encoder",
        "source_model_key_prefix": "", "source_model_key_patterns": list(TEXT_ENCODER_KEYS)}}
    (run / "config.yaml").write_text(yaml.safe_dump(config))

    spec = inspect_artifact(run / "checkpoints" / "iter_000000002")
    assert spec.iteration == 2 and spec.prompt_pixel_frames == 9 and spec.lora is None
    assert spec.student[-1].prefix == "net" and spec.text[0].path == released.resolve()
    assert spec.tokenizer_path == (run / "released" / "text_tokenizer").resolve()
    seen = []
    artifact = load_artifact(spec, device="cpu", dtype=torch.float32, progress=lambda *a: seen.append(a))
    assert [s[0] for s in seen] == ["und", "und", "student", "student"]
    assert all(torch.equal(a, b) for a, b in zip(text.state_dict().values(),
                                                 artifact.context_encoder.state_dict().values()))
    assert not any(p.requires_grad for p in artifact.student.parameters())
    assert artifact.report["iteration"] == 2 and artifact.special_tokens == spec.config.special_tokens

    exported = save_artifact(artifact, tmp_path / "export")
    again = inspect_artifact(exported / "student.safetensors")  # a file inside the export also works
    assert again.checkpoint == exported and again.iteration == 2
    second = load_artifact(again, device="cpu", dtype=torch.float32)
    for a, b in ((artifact.student, second.student), (artifact.context_encoder, second.context_encoder)):
        assert all(torch.equal(x, y) for x, y in zip(a.state_dict().values(), b.state_dict().values()))

    manifest = exported / "manifest.json"
    manifest.write_text(manifest.read_text().replace('"version": 1', '"version": 7'))
    with pytest.raises(ValueError):
        inspect_artifact(exported)
    with pytest.raises(FileNotFoundError):
        inspect_artifact(tmp_path / "nowhere")


def test_undeclared_lora_tensors_are_refused(tmp_path):
    from agentgarten_b200.inference.cosmos3 import WeightSource, _TowerLoader
    module = torch.nn.Linear(4, 4, bias=False)
    tensor_file.write_tensors({"weight": torch.zeros(4, 4), "weight.lora_A": torch.zeros(2, 4)},
                              tmp_path / "w.safetensors")
    with pytest.raises(ValueError, match="undeclared LoRA"):
        _TowerLoader(module, (WeightSource(pathlib.Path(tmp_path / "w.safetensors"), ""),)).run()
