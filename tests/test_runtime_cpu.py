"""Unit tests of runtime pieces on CPU: RNG capture/restore, loader resume, LR lambdas,
gradient clipping, LoRA injection, geometry preprocessing, media helpers."""

import math
import pickle
import random

import numpy as np
import pytest
import torch

from agentgarten_b200.data.loader import StatefulDataLoader
from agentgarten_b200.data.video import SyntheticLatentDataset, SyntheticVideoDataset
from agentgarten_b200.infra import rng_state
from agentgarten_b200.infra.callbacks.grad_clip import clip_grad_norm_, clip_grad_norm_groups_
from agentgarten_b200.infra.callbacks.media import media_artifact_filename, video_batch_to_cpu_uint8
from agentgarten_b200.infra.optim import CosineDecay, LinearWarmup, LinearWarmupCosineDecay
from agentgarten_b200.networks.cosmos3 import geometry
from agentgarten_b200.networks.lora import LORA_PARAMETER_PATTERN, LoRALinear, initialize_lora_parameters, inject_lora


# ----------------------------------------------------------------------------- RNG
def _draw():
    return random.random(), float(np.random.rand()), float(torch.rand(1))


def test_rng_capture_restore_and_isolation():
    random.seed(1); np.random.seed(2); torch.manual_seed(3)
    state = rng_state.capture_distributed_rng_state()
    rng_state.validate_distributed_rng_state(state)
    first = _draw()
    with rng_state.isolated_rng():
        torch.manual_seed(99); random.seed(99); np.random.seed(99)
        _draw()
    second = _draw()  # the block above left no trace
    rng_state.restore_distributed_rng_state(state)
    assert _draw() == first and _draw() == second


def test_rng_blob_refuses_foreign_pickles():
    random.seed(5)
    state = rng_state.capture_distributed_rng_state()
    key = next(k for k in state["ranks"])
    evil = pickle.dumps(print)  # a global that is not a NumPy reconstructor
    tampered = {**state, "ranks": {key: {**state["ranks"][key],
                                         "python_blob": torch.tensor(list(evil), dtype=torch.uint8),
                                         "python_length": len(evil)}}}
    with pytest.raises(Exception):
        rng_state.validate_distributed_rng_state(tampered)
    wrong_world = {**state, "world_size": 7}
    with pytest.raises(RuntimeError):
        rng_state.validate_distributed_rng_state(wrong_world)


# -------------------------------------------------------------------------- loader
def _ids(batches):
    return [b["sample_id"].tolist() for b in batches]


def test_loader_resumes_mid_epoch_and_across_epochs():
    data = SyntheticLatentDataset(length=10, latent_frames=1, latent_height=2, latent_width=2,
                                  channels=4, text_tokens=3, vocab_size=50)
    make = lambda: StatefulDataLoader(data, batch_size=2, shuffle=True, seed=11, pin_memory=False)  # noqa: E731
    straight = make()
    epoch0 = _ids(list(straight))
    epoch1 = _ids(list(straight))
    assert len(epoch0) == 5 and sorted(sum(epoch0, [])) == list(range(10)) and epoch0 != epoch1
    assert straight.state_dict() == {"epoch": 2, "batch_offset": 0}

    stopped = make()
    iterator = iter(stopped)
    head = _ids([next(iterator), next(iterator)])
    cursor = stopped.state_dict()
    assert cursor == {"epoch": 0, "batch_offset": 2}
    resumed = make()
    resumed.load_state_dict(cursor)
    assert head + _ids(list(resumed)) == epoch0
    assert _ids(list(resumed)) == epoch1
    # an older iterator may not advance the cursor once a newer one exists
    stale = iter(stopped)
    iter(stopped)
    with pytest.raises(RuntimeError):
        next(stale)
    with pytest.raises(ValueError):
        resumed.load_state_dict({"epoch": -1, "batch_offset": 0})
    assert make().resume_signature() == straight.resume_signature()


def test_synthetic_video_dataset_is_seeded():
    data = SyntheticVideoDataset(length=3, num_frames=5, height=8, width=8)
    a, b = data[1], data[1]
    assert all(torch.equal(a[k], b[k]) for k in a if torch.is_tensor(a[k]))
    assert not torch.equal(data[0]["video"], data[1]["video"])


# ------------------------------------------------------------------------------ LR
def test_lr_lambdas():
    warm = LinearWarmup(warmup_steps=4, start_factor=0.2)
    assert warm(0) == pytest.approx(0.2) and warm(2) == pytest.approx(0.6) and warm(4) == 1.0 and warm(99) == 1.0
    cosine = CosineDecay(decay_steps=10, min_factor=0.1)
    assert cosine(0) == pytest.approx(1.0) and cosine(10) == pytest.approx(0.1) and cosine(50) == pytest.approx(0.1)
    assert cosine(5) == pytest.approx(0.1 + 0.9 * 0.5)
    both = LinearWarmupCosineDecay(warmup_steps=2, decay_steps=12, start_factor=0.0, min_factor=0.0)
    values = [both(s) for s in range(13)]
    assert values[0] == 0.0 and values[2] == pytest.approx(1.0) and values[12] == pytest.approx(0.0, abs=1e-9)
    assert all(a >= b - 1e-12 for a, b in zip(values[2:], values[3:]))
    pickle.loads(pickle.dumps(both))  # schedulers are checkpointed by value
    # keyword names, defaults and validation of a resolved reference config
    default = LinearWarmup()
    assert (default.warmup_steps, default.start_factor) == (100, 1.0e-6) and default(0) > 0.0
    with pytest.raises(TypeError):
        LinearWarmup(4)
    for bad in (dict(decay_steps=0), dict(decay_steps=5, min_factor=1.5), dict(decay_steps=5, min_factor=float("nan"))):
        with pytest.raises(ValueError):
            CosineDecay(**bad)
    for bad in (dict(warmup_steps=-1, decay_steps=5), dict(warmup_steps=5, decay_steps=5),
                dict(warmup_steps=1, decay_steps=5, start_factor=2.0)):
        with pytest.raises(ValueError):
            LinearWarmupCosineDecay(**bad)


# ------------------------------------------------------------------------ clipping
def test_group_clip_matches_torch_and_observe_only():
    torch.manual_seed(0)
    a, b = torch.nn.Parameter(torch.randn(5, 3)), torch.nn.Parameter(torch.randn(7))
    a.grad, b.grad = torch.randn(5, 3), torch.randn(7)
    want = math.sqrt(float(a.grad.square().sum() + b.grad.square().sum()))
    before = a.grad.clone()
    total, roles = clip_grad_norm_groups_({"student": [a], "critic": [b, a]}, float("inf"))
    assert float(total) == pytest.approx(want, rel=1e-6) and set(roles) == {"student", "critic"}
    assert torch.equal(a.grad, before)  # inf: observe only; `a` counted once
    total = clip_grad_norm_([a, b], 0.5)
    after = math.sqrt(float(a.grad.square().sum() + b.grad.square().sum()))
    assert float(total) == pytest.approx(want, rel=1e-6) and after == pytest.approx(0.5, rel=1e-4)
    with pytest.raises(ValueError):
        clip_grad_norm_([a], -1.0)


# ---------------------------------------------------------------------------- LoRA
def test_lora_injection_targets_and_identity_at_init():
    import re

    torch.manual_seed(0)
    net = torch.nn.ModuleDict({"layers": torch.nn.ModuleList([
        torch.nn.ModuleDict({"q": torch.nn.Linear(8, 8, bias=False), "mlp": torch.nn.Linear(8, 16)})
        for _ in range(2)])})
    x = torch.randn(3, 8)
    plain = net["layers"][0]["q"](x)
    names = inject_lora(net, {"rank": 2, "alpha": 2.0, "dropout": 0.0,
                              "module_patterns": [r"layers\.\d+\.q"]})
    assert sorted(names) == ["layers.0.q", "layers.1.q"]
    assert isinstance(net["layers"][0]["q"], LoRALinear) and not isinstance(net["layers"][0]["mlp"], LoRALinear)
    initialize_lora_parameters(net, seed=0)
    assert torch.allclose(net["layers"][0]["q"](x), plain)  # B starts at zero
    adapters = [n for n, _ in net.named_parameters() if re.fullmatch(LORA_PARAMETER_PATTERN, n)]
    assert len(adapters) == 4
    assert inject_lora(net, {"rank": 2, "alpha": 2.0, "dropout": 0.0,
                             "module_patterns": [r"nothing\.matches"]}) == ()
    with pytest.raises(ValueError):
        inject_lora(net, {"rank": 0, "module_patterns": [r".*"]})


# ------------------------------------------------------------------------ geometry
def test_depth_colours_and_normals():
    depth = torch.tensor([0.0, float("nan"), 0.5, 5.0, 1e6]).view(1, 1, 1, 1, 5)
    rgb = geometry.colorize_depth(depth, torch.tensor([1.0]))
    assert rgb.shape == (1, 3, 1, 1, 5) and rgb.min() >= 0 and rgb.max() <= 1
    assert torch.equal(rgb[0, :, 0, 0, 0], torch.zeros(3)) and torch.equal(rgb[0, :, 0, 0, 1], torch.zeros(3))
    assert torch.allclose(rgb[0, :, 0, 0, 4], torch.ones(3), atol=1e-3)  # far end of the walk is white
    near, far = rgb[0, :, 0, 0, 2], rgb[0, :, 0, 0, 3]
    assert near.sum() < far.sum()
    raw = torch.tensor([[255, 127, 127], [127, 127, 127]], dtype=torch.uint8).t().reshape(1, 3, 1, 1, 2)
    unit = geometry.prepare_normal(raw)
    assert torch.allclose(unit[0, :, 0, 0, 0].norm(), torch.tensor(1.0), atol=1e-5)
    assert float(unit[0, :, 0, 0, 1].abs().max()) <= 1.0
    floats = torch.randn(1, 3, 1, 2, 2)
    assert torch.equal(geometry.prepare_normal(floats), floats)
    with pytest.raises(TypeError):
        geometry.prepare_normal(torch.zeros(1, 3, 1, 2, 2, dtype=torch.int32))
    low = geometry.downsample_geometry({"depth": torch.arange(16.0).view(1, 1, 1, 4, 4)}, factor=2)["depth"]
    assert low.shape == (1, 1, 1, 2, 2) and float(low[0, 0, 0, 0, 0]) == pytest.approx(2.5)


def test_geometry_config_validation_and_stretch():
    with pytest.raises(ValueError):
        geometry.GeometryAugmentationConfig(modality_dropout_probability=1.5)
    videos = {"depth": torch.rand(1, 3, 2, 30, 52), "normal": torch.rand(1, 3, 2, 30, 52)}
    out = geometry.stretch_geometry(videos, training=False, divisor=32)
    assert all(v.shape[-2] % 32 == 0 and v.shape[-1] % 32 == 0 for v in out.values())


# --------------------------------------------------------------------------- media
def test_media_names_and_uint8_conversion():
    name = media_artifact_filename(artifact_name="comparison grid", iteration=12, rank=3,
                                   sample_batch_index=1, extension="mp4", batch_index=0)
    assert name == "Iter000000012_Rank0003_comparison_grid01_00.mp4"
    wide = media_artifact_filename(artifact_name="x", iteration=1, rank=0, sample_batch_index=120, extension="jpg")
    assert "@120" in wide
    video = torch.stack([torch.full((3, 2, 4, 4), -1.0), torch.full((3, 2, 4, 4), 1.0)])
    frames = video_batch_to_cpu_uint8(video, layout="BCTHW", float_range="minus_one_one")
    assert frames.shape == (2, 3, 2, 4, 4) and frames.dtype == torch.uint8 and frames.device.type == "cpu"
    assert int(frames[0].max()) == 0 and int(frames[1].min()) == 255


def test_manifest_dataset_reads_validates_and_signs(tmp_path):
    import json

    from agentgarten_b200.data.video import ManifestVideoDataset

    frames, height, width = 5, 8, 12
    rng = np.random.default_rng(0)
    rows = []
    for index in range(2):
        np.save(tmp_path / f"clip{index}.npy", rng.integers(0, 255, (frames, height, width, 3), dtype=np.uint8))
        np.save(tmp_path / f"depth{index}.npy", rng.random((frames, height, width), dtype=np.float32) + 0.1)
        np.save(tmp_path / f"normal{index}.npy", rng.standard_normal((frames, height, width, 3)).astype(np.float32))
        rows.append({"video": f"clip{index}.npy", "depth": f"depth{index}.npy", "normal": f"normal{index}.npy",
                     "caption": f"clip number {index}", "depth_scale": 2.0})
    manifest = tmp_path / "train.jsonl"
    manifest.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    data = ManifestVideoDataset(str(manifest), num_frames=frames, height=height, width=width, fps=16.0)
    assert len(data) == 2
    item = data[1]
    assert item["video"].shape == (frames, 3, height, width) and item["video"].dtype == torch.uint8
    assert item["depth"].shape == (frames, 1, height, width) and item["normal"].shape == (frames, 3, height, width)
    assert torch.allclose(item["normal"].norm(dim=1), torch.ones(frames, height, width), atol=1e-5)
    assert item["caption"] == "clip number 1" and item["depth_scale"] == 2.0 and item["sample_id"] == 1
    signature = data.resume_signature()
    manifest.write_text(manifest.read_text() + json.dumps(rows[0]) + "\n")
    assert ManifestVideoDataset(str(manifest), num_frames=frames, height=height, width=width).resume_signature() != signature
    # wrong length and bad values are refused with the file name
    with pytest.raises(ValueError, match="clip0.npy"):
        ManifestVideoDataset(str(manifest), num_frames=frames + 4, height=height, width=width)[0]
    bad = np.load(tmp_path / "depth0.npy"); bad[0, 0, 0] = -1.0
    np.save(tmp_path / "depth0.npy", bad)
    with pytest.raises(ValueError, match="non-negative"):
        data[0]


def test_encoded_video_is_decoded_by_the_available_backend(tmp_path):
    cv2 = pytest.importorskip("cv2")
    from agentgarten_b200.data.video import _read_video

    path = tmp_path / "clip.avi"
    writer = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"MJPG"), 16.0, (16, 8))
    if not writer.isOpened():
        pytest.skip("no video encoder in this OpenCV build")
    for value in (0, 120, 250):
        writer.write(np.full((8, 16, 3), value, dtype=np.uint8))
    writer.release()
    frames = _read_video(path)
    assert frames.shape == (3, 3, 8, 16) and frames.dtype == torch.uint8
    assert abs(int(frames[1].float().mean()) - 120) < 6


def test_keep_plan_recomputes_on_cpu_and_obeys_the_switch(monkeypatch):
    """Off the GPU every layer of the operator-by-operator path is recomputed; the switch
    fixes the choice wherever the layers run."""
    import torch

    from agentgarten_b200.ops import fused_layer
    from agentgarten_b200.parallel.engine import _KeepPlan

    plan = _KeepPlan()
    chunks = [torch.zeros(1, 4, 8)]
    args = (chunks, None, None, 0, None)
    assert plan.keeps(object(), args) is False
    monkeypatch.setattr(fused_layer, "_KEEP_MODE", "never")
    assert plan.keeps(object(), args) is False
    monkeypatch.setattr(fused_layer, "_KEEP_MODE", "always")
    assert plan.keeps(object(), args) is False  # CPU tensors: nothing to measure, recompute


def test_peer_exchange_declines_what_it_cannot_serve(monkeypatch):
    """CPU tensors, a switched-off path and an uninitialised process group fall through to the
    library collective (the function returns None and allocates nothing)."""
    import torch

    from agentgarten_b200.parallel import peer_exchange

    value = torch.zeros(2, 4, 8)
    assert peer_exchange.exchange(value, None) is None
    monkeypatch.setenv("AGB200_NCCL_EXCHANGE", "1")
    assert peer_exchange.exchange(value, None) is None
    assert not peer_exchange._links
    peer_exchange.release()


def test_parallel_config_refuses_what_the_engine_cannot_honour():
    """Knobs of the reference's FSDP2 wrapping that would change behaviour are refused, not
    ignored; the ones that cannot matter here are accepted."""
    from agentgarten_b200.parallel.engine import ParallelConfig, replicated_parameter_bytes

    ParallelConfig(reshard_after_forward=True)
    ParallelConfig(reshard_after_forward=False, fsdp_mesh_shape=(2, 8))
    with pytest.raises(ValueError, match="float32"):
        ParallelConfig(reduce_dtype="bfloat16")
    with pytest.raises(ValueError, match="fsdp_mesh_shape"):
        ParallelConfig(fsdp_mesh_shape=(2, 2, 2))
    with pytest.raises(ValueError, match="one node"):
        ParallelConfig(fsdp_mesh_shape=(1, 16))
    tower = torch.nn.Sequential(torch.nn.Linear(8, 8, bias=False), torch.nn.Linear(8, 4, bias=False))
    tower[1].requires_grad_(False)
    assert replicated_parameter_bytes(tower) == 2 * (64 * 2) + 32 * 2


def test_poison_fills_data_buffers_only_when_asked(monkeypatch):
    from agentgarten_b200.parallel import debug

    monkeypatch.delenv("AGB200_POISON", raising=False)
    rows = torch.zeros(4, 8, dtype=torch.bfloat16)
    assert debug.poison(rows) is rows and rows.abs().sum() == 0
    monkeypatch.setenv("AGB200_POISON", "1")
    assert torch.isnan(debug.poison(rows)).all()
    assert torch.isnan(debug.poison(torch.zeros(3, dtype=torch.float32))).all()
    assert debug.poison(torch.zeros(0)).numel() == 0


def test_switch_share_declines_off_the_gpu_and_pads_to_whole_vectors():
    """Without a process group, on CPU tensors or with the switch path switched off, the callers
    keep their library collective; payloads are handed to the kernel in whole 16-byte vectors."""
    from agentgarten_b200.parallel import switch_share

    rows = torch.arange(21, dtype=torch.float32).reshape(3, 7)
    assert switch_share.all_gather(rows) is None
    assert switch_share.broadcast(rows, 0) is False
    padded = switch_share._bytes_of(rows.to(torch.bfloat16))
    assert padded.dtype == torch.uint8 and padded.numel() == 48 and padded.data_ptr() % 16 == 0
    assert torch.equal(padded[:42].view(torch.bfloat16), rows.to(torch.bfloat16).reshape(-1))
    whole = switch_share._bytes_of(torch.zeros(8, dtype=torch.float32))
    assert whole.numel() == 32
    assert switch_share._round_up(17, 16) == 32 and switch_share._round_up(32, 16) == 32


def test_wandb_sinks_share_one_lazily_started_run(monkeypatch):
    """A stand-in for the SDK records the calls: nothing happens before the first write, both
    sinks log into one run, x-axes are declared once, media keys follow
    ``<split>/batch_<index>/<artifact>``, the last close finishes the run, an asynchronous sink
    survives a failing service, and a missing SDK is an error that names the extra."""
    import sys
    import types

    from agentgarten_b200.infra.callbacks import wandb as sinks

    calls = []
    fake = types.ModuleType("wandb")
    fake.run = None

    def init(**kwargs):
        calls.append(("init", kwargs))
        fake.run = object()

    def finish():
        calls.append(("finish",))
        fake.run = None

    fake.init, fake.finish = init, finish
    fake.login = lambda **kwargs: calls.append(("login", kwargs))
    fake.define_metric = lambda pattern, step_metric: calls.append(("axis", pattern, step_metric))
    fake.log = lambda payload, step: calls.append(("log", dict(payload), step))
    fake.Image = lambda array: ("image", tuple(array.shape))
    fake.Video = lambda data, format: ("video", format)
    monkeypatch.setitem(sys.modules, "wandb", fake)
    monkeypatch.setenv("WANDB_API_KEY", "k")

    metrics = sinks.WandbMetricSink("proj", "grp", "run-1", "offline", step_metrics={"val/*": "val/step"})
    media = sinks.WandbArtifactWriter("proj", group="grp", name="run-1", mode="offline", fps=4)
    assert calls == [] and metrics.step_metrics == {"val/*": "val/step"} and media.fps == 4
    metrics.write({"train/loss": 1.5}, iteration=3)
    assert [c[0] for c in calls] == ["login", "init", "axis", "log"]
    assert calls[1][1] == {"project": "proj", "group": "grp", "name": "run-1", "mode": "offline"}
    assert calls[3] == ("log", {"train/loss": 1.5}, 3)
    clip = torch.zeros(2, 3, 2, 8, 8)
    media.write({"sample": clip, "still": torch.zeros(3, 1, 8, 8)}, output_dir="unused", split="validation",
                iteration=4, rank=0, sample_batch_index=7)
    assert [c[0] for c in calls].count("init") == 1
    logged = calls[-1]
    assert logged[0] == "log" and logged[2] == 4
    assert set(logged[1]) == {"validation/batch_0007/sample/000", "validation/batch_0007/sample/001",
                              "validation/batch_0007/still"}
    assert logged[1]["validation/batch_0007/sample/000"] == ("video", "mp4")
    assert logged[1]["validation/batch_0007/still"][0] == "image"
    metrics.close()
    assert ("finish",) not in calls          # the media writer still holds the run
    media.close()
    assert calls[-1] == ("finish",)
    metrics.write({"train/loss": 2.0}, iteration=5)   # closed sinks stay quiet
    assert calls[-1] == ("finish",)

    # asynchronous writes: a service that fails once silences the sink, close() still returns
    fake.log = lambda payload, step: (_ for _ in ()).throw(ConnectionError("service down"))
    background = sinks.WandbMetricSink("proj", async_write=True)
    background.write({"a": 1.0}, iteration=1)
    background.write({"a": 2.0}, iteration=2)
    background.close()
    assert isinstance(background._worker_error, ConnectionError) and fake.run is None
    background.write({"a": 3.0}, iteration=3)

    monkeypatch.setitem(sys.modules, "wandb", None)    # import wandb -> ModuleNotFoundError
    import pytest

    with pytest.raises(ModuleNotFoundError, match=r"wm\[wandb\]"):
        sinks.WandbMetricSink("proj").write({"a": 1.0}, iteration=1)
