"""Outputs of the package's pure and seeded functions, for differential tests.

The same file runs against either tree: with ``PYTHONPATH=baseline/_ref:baseline/shims`` the
imports below resolve to the unmodified reference package, inside this repository they resolve
to the ``wm`` alias of this package.  ``collect()`` returns ``{name: tensor | number | list}``;
as a script it writes that dictionary with ``torch.save``.  Every section is independent: a
section that cannot run in one tree records ``"<section>/error"`` instead of stopping the rest.

Covered: rectified-flow utilities and the UniPC solver, learning-rate factors, geometry
preprocessing and its seeded augmentations, media conversion and file names, the history window,
the phase clock of the distillation recipe, the stream position policy, seeded initialisation of
the discriminator head and of LoRA adapters, the synthetic dataset and the stateful loader, a
whole ``Trainer.train`` run on a toy model with the clip / spike monitor and the metric callback,
the tiny decoders (parallel, sequential, streamed), streams in all three position modes with
eviction, a prompt change and reference images, ``sample()`` of the three objectives, raw batches
through the conditioner, periodic sampling with the media writer's files and rules, the codec wrapper's surface, the
objective base class, bounded history windows, weight overlays at start-up, the optimizer's CPU path, constants and recipe trees, utilities,
clipping helpers, lazy calls, the metric callback's corner cases, resume under a changed recipe,
and the Wan 2.2 VAE (encode / decode of a small clip with shared random weights).
"""

from __future__ import annotations

import sys

import torch


def _flow(out: dict) -> None:
    from wm.models.flow import (FlowUniPC, RectifiedFlowSchedule, UniformShift, invariant_randn,
                                rf_interpolate, rf_x0, sampling_seeds, shift_sigma)

    grid = torch.linspace(0.0, 1.0, 11)
    out["flow/shift_sigma"] = shift_sigma(grid, 5.0)
    g = torch.Generator().manual_seed(3)
    clean, noise = torch.randn(2, 4, 3, 5, 6, generator=g), torch.randn(2, 4, 3, 5, 6, generator=g)
    for label, sigma in (("per_sample", torch.tensor([0.25, 0.8])),
                         ("per_frame", torch.tensor([[0.1, 0.5, 0.9], [0.3, 0.3, 0.7]]))):
        noisy = rf_interpolate(clean, noise, sigma)
        out[f"flow/interpolate/{label}"] = noisy
        out[f"flow/x0/{label}"] = rf_x0(noisy, sigma, noise - clean)
    for kind in ("uniform", "logitnormal", "waver"):
        schedule = RectifiedFlowSchedule(shift=5.0, train_distribution=kind)
        out[f"flow/schedule/{kind}"] = schedule.sample((4, 3), device=torch.device("cpu"),
                                                       generator=torch.Generator().manual_seed(11))
    out["flow/uniform_shift"] = UniformShift(3.0).sample(6, device=torch.device("cpu"),
                                                         generator=torch.Generator().manual_seed(12))
    out["flow/invariant_randn/0"] = invariant_randn(clean, [7, 8])
    out["flow/invariant_randn/2"] = invariant_randn(clean, [7, 8], stream=2)
    out["flow/seeds/ids"] = sampling_seeds({"latent": clean, "sample_id": torch.tensor([40, 2])}, 5)
    out["flow/seeds/plain"] = sampling_seeds({"latent": clean}, 5)
    solver = FlowUniPC(6, shift=5.0)
    out["flow/unipc/sigmas"] = solver.sigmas
    out["flow/unipc/timesteps"] = solver.timesteps
    target = torch.randn(clean.shape, generator=g)

    def field(sample, sigma):   # the exact velocity towards `target` under the linear path
        return (sample - target) / max(sigma, 1e-3)

    out["flow/unipc/run"] = solver.run(noise.clone(), field, post_step=lambda x: x.clamp(-4, 4))


def _lr(out: dict) -> None:
    from wm.infra.optim import CosineDecay, LinearWarmup, LinearWarmupCosineDecay

    steps = (0, 1, 5, 49, 50, 99, 100, 101, 500, 999, 1000, 5000)
    factors = {"warmup": LinearWarmup(warmup_steps=100, start_factor=0.1),
               "cosine": CosineDecay(decay_steps=1000, min_factor=0.05),
               "both": LinearWarmupCosineDecay(warmup_steps=50, decay_steps=1000, start_factor=0.0,
                                               min_factor=0.1)}
    for name, factor in factors.items():
        out[f"lr/{name}"] = [float(factor(step)) for step in steps]


def _geometry(out: dict) -> None:
    from wm.networks.cosmos3 import geometry

    g = torch.Generator().manual_seed(21)
    depth = torch.rand(2, 1, 3, 24, 40, generator=g) * 30.0
    depth[0, 0, 0, 0, 0] = float("nan")
    depth[1, 0, 1, 2, 3] = 0.0
    scale = torch.tensor([1.0, 2.5])
    out["geometry/colorize"] = geometry.colorize_depth(depth, scale)
    raw = torch.randint(0, 256, (2, 3, 3, 24, 40), generator=g, dtype=torch.uint8)
    raw[0, :, 0, 0, 0] = 128
    out["geometry/normal/uint8"] = geometry.prepare_normal(raw)
    out["geometry/normal/float"] = geometry.prepare_normal(torch.randn(1, 3, 2, 4, 4, generator=g))
    videos = {"depth": torch.randn(2, 3, 3, 24, 40, generator=g), "normal": torch.randn(2, 3, 3, 24, 40, generator=g)}
    videos["depth"][0, 0, 0, 0, 0] = float("inf")
    low = geometry.downsample_geometry(videos, factor=4)
    for name, value in low.items():
        out[f"geometry/downsample/{name}"] = value
    clean = {name: torch.nan_to_num(value, posinf=0.0) for name, value in videos.items()}
    for training in (False, True):
        torch.manual_seed(5)
        grown = geometry.stretch_geometry(clean, training=training, divisor=32)
        for name, value in grown.items():
            out[f"geometry/stretch/{'train' if training else 'eval'}/{name}"] = value
    config = geometry.GeometryAugmentationConfig(
        modality_dropout_probability=0.5, spatial_probability=1.0, spatial_max_scale=1.2,
        spatial_max_shift_fraction=0.05, spatial_max_shear=0.05, spatial_max_perspective=0.05,
        texture_suppression_probability=1.0, texture_downsample_min=1.5, texture_downsample_max=3.0)
    batch = {"sample_id": [3, 9], "geometry_condition_is_augmented": [False, False]}
    for training in (True, False):
        torch.manual_seed(6)
        changed = geometry.augment_geometry(clean, data_batch=batch, training=training, config=config)
        for name, value in changed.items():
            out[f"geometry/augment/{'train' if training else 'eval'}/{name}"] = value
    torch.manual_seed(7)
    jitter = {"depth_scale": torch.tensor([1.0, 2.0]), "depth_scale_jitter_eligible": torch.tensor([True, False]),
              "depth_scale_jitter_bounds": torch.tensor([[0.5, 2.0], [0.5, 2.0]])}
    out["geometry/depth_scale/train"] = geometry.depth_scale(jitter, training=True, batch_size=2)
    out["geometry/depth_scale/eval"] = geometry.depth_scale(jitter, training=False, batch_size=2)


def _media(out: dict) -> None:
    from wm.infra.callbacks.media import media_artifact_filename, video_batch_to_cpu_uint8

    g = torch.Generator().manual_seed(31)
    clip = torch.rand(2, 3, 5, 6, 8, generator=g) * 2.4 - 1.2
    out["media/minus_one_one"] = video_batch_to_cpu_uint8(clip, frame_chunk_size=2)
    out["media/zero_one"] = video_batch_to_cpu_uint8(clip.permute(0, 2, 1, 3, 4), layout="BTCHW",
                                                     float_range="zero_one")
    out["media/names"] = [
        media_artifact_filename(artifact_name="grid 2x2/ü", iteration=12, rank=3, sample_batch_index=1,
                                extension="mp4", batch_index=0),
        media_artifact_filename(artifact_name="..", iteration=1, rank=0, sample_batch_index=120, extension="jpg"),
        media_artifact_filename(artifact_name="a.b-c_d", iteration=10**9, rank=12345, sample_batch_index=7,
                                extension="png", batch_index=101)]


def _policies(out: dict) -> None:
    from wm.models.dmd import PhaseClock
    from wm.networks.cosmos3.streaming import StreamPolicy
    from wm.protocols import HistoryWindow

    blocks = list(range(9))
    out["history/all"] = HistoryWindow().visible(blocks)
    out["history/sink1_recent3"] = HistoryWindow(sink_blocks=1, recent_blocks=3).visible(blocks)
    out["history/recent0"] = HistoryWindow(sink_blocks=2, recent_blocks=0).visible(blocks)
    clock = PhaseClock(fake_score_updates_per_student=3, warmup_updates=2)
    span = range(0, 30)
    out["clock/student"] = [bool(clock.is_student(i)) for i in span]
    out["clock/warmup"] = [bool(clock.is_warmup(i)) for i in span]
    out["clock/updates"] = [sorted(clock.role_updates(i).items()) for i in span]
    out["clock/due2"] = [bool(clock.is_cadence_due(i, 2)) for i in span]
    for rope in ("absolute", "contiguous", "top_aligned"):
        policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, rope=rope, train_frames=21)
        for first, count, cached in ((0, 1, 0), (1, 4, 1), (9, 4, 9), (29, 4, 9)):
            try:
                out[f"stream/{rope}/{first}"] = policy.positions(first, count, cached)
            except Exception as error:   # the same refusal must come from both trees
                out[f"stream/{rope}/{first}"] = f"{type(error).__name__}"


def _seeded_modules(out: dict) -> None:
    from wm.networks.discriminator import DiscriminatorHead
    from wm.networks.lora import initialize_lora_parameters, inject_lora

    head = DiscriminatorHead(hidden_size=32, feature_layers=(1, 3), mlp_ratio=2.0, num_heads=4, seed=123)
    for name, value in head.state_dict().items():
        out[f"discriminator/state/{name}"] = value
    g = torch.Generator().manual_seed(41)
    features = [[torch.randn(2, 7, 32, generator=g), torch.randn(2, 7, 32, generator=g)]]
    out["discriminator/logits"] = head(features).detach()
    flipped = DiscriminatorHead(hidden_size=32, feature_layers=(1, 3), mlp_ratio=2.0, num_heads=4, seed=123,
                                initial_logit_sign=-1.0)
    out["discriminator/flipped"] = flipped(features).detach()

    class Tower(torch.nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.to_q = torch.nn.Linear(16, 16, bias=False)
            self.to_out = torch.nn.Linear(16, 16)
            self.other = torch.nn.Linear(16, 4)

    torch.manual_seed(9)
    tower = Tower()
    replaced = inject_lora(tower, {"rank": 4, "alpha": 8.0, "dropout": 0.0, "target_modules": ["to_q", "to_out"]})
    out["lora/replaced"] = list(replaced)
    initialize_lora_parameters(tower, seed=77)
    for name, value in tower.state_dict().items():
        out[f"lora/state/{name}"] = value
    out["lora/forward"] = tower.to_out(tower.to_q(torch.ones(3, 16))).detach()


def _data(out: dict) -> None:
    from wm.data.loader import StatefulDataLoader
    from wm.data.video import SyntheticVideoDataset

    dataset = SyntheticVideoDataset(length=11, num_frames=3, height=8, width=12, fps=12.0)
    sample = dataset[4]
    for key, value in sample.items():
        out[f"data/sample/{key}"] = value
    out["data/length"] = len(dataset)

    class Indices(torch.utils.data.Dataset):
        def __len__(self) -> int:
            return 11

        def __getitem__(self, index: int):
            return {"index": torch.tensor(index)}

    def order(loader, count):
        seen, iterator = [], iter(loader)
        for _ in range(count):
            try:
                seen.append(next(iterator)["index"].tolist())
            except StopIteration:
                seen.append("end")
                iterator = iter(loader)
        return seen

    loader = StatefulDataLoader(Indices(), batch_size=2, shuffle=True, seed=5, num_workers=0, pin_memory=False)
    out["data/len"] = len(loader)
    out["data/signature"] = sorted((k, str(v)) for k, v in loader.resume_signature().items())
    out["data/order"] = order(loader, 9)
    cursor = dict(loader.state_dict())
    out["data/cursor"] = sorted(cursor.items())
    resumed = StatefulDataLoader(Indices(), batch_size=2, shuffle=True, seed=5, num_workers=0, pin_memory=False)
    resumed.load_state_dict(cursor)
    out["data/resumed"] = order(resumed, 4)
    out["data/continued"] = order(loader, 4)
    wrapped = StatefulDataLoader(Indices(), batch_size=2, shuffle=False, seed=5, num_workers=0, pin_memory=False,
                                 drop_last=False)
    wrapped.load_state_dict({"epoch": 1, "batch_offset": 8})
    out["data/wrapped_cursor"] = sorted(wrapped.state_dict().items())
    out["data/keep_last"] = order(wrapped, 7)


def _training_loop(out: dict) -> None:
    import json
    import tempfile
    from pathlib import Path

    from wm.data.loader import StatefulDataLoader
    from wm.infra.callbacks import CallbackGroup, GradClipMonitor, ScalarMetricCallback
    from wm.infra.model import Model
    from wm.infra.optim import LinearWarmup
    from wm.infra.trainer import Trainer

    class Toy(Model):
        def __init__(self) -> None:
            super().__init__(optimizer_parameter_groups=[{"patterns": r".*\.bias", "lr": 0.05}])
            g = torch.Generator().manual_seed(61)
            self.body, self.head = torch.nn.Linear(6, 4), torch.nn.Linear(4, 1)
            with torch.no_grad():
                for parameter in self.parameters():
                    parameter.copy_(torch.randn(parameter.shape, generator=g) * 0.5)

        def parallelize(self, device) -> None:
            return None

        def _score(self, batch):
            error = self.head(torch.tanh(self.body(batch["x"]))) - batch["y"]
            loss = error.square().mean()
            return {"metrics/mse": loss.detach(), "metrics/abs": error.abs().mean().detach(),
                    "note": "not a metric"}, loss

        def training_step(self, data_batch, iteration):
            return self._score(data_batch)

        def validation_step(self, data_batch, iteration):
            return self._score(data_batch)

        def sample(self, data_batch, **sampling_options):
            return {}

    class Rows(torch.utils.data.Dataset):
        def __init__(self, count: int, seed: int) -> None:
            g = torch.Generator().manual_seed(seed)
            self.x, self.y = torch.randn(count, 6, generator=g), torch.randn(count, 1, generator=g) * 3.0

        def __len__(self) -> int:
            return len(self.x)

        def __getitem__(self, index: int):
            return {"x": self.x[index], "y": self.y[index], "sample_index": index}

    class Sink:
        def __init__(self) -> None:
            self.rows = []

        def write(self, metrics, *, iteration):
            self.rows.append((int(iteration), sorted((str(k), float(v)) for k, v in metrics.items())))

    model, sink = Toy(), Sink()
    groups = model._group_trainable_parameters()
    out["loop/groups"] = [(sorted(k for k in group if k != "params"), [tuple(p.shape) for p in group["params"]])
                          for group in groups]
    optimizer = torch.optim.SGD(groups, lr=0.2, momentum=0.5)
    scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, lr_lambda=LinearWarmup(warmup_steps=4, start_factor=0.25))
    model.optimizer_dict, model.scheduler_dict = {"net": optimizer}, {"net": scheduler}
    with tempfile.TemporaryDirectory() as scratch:
        monitor = GradClipMonitor(max_norm=0.75, spike_threshold=2.0, spike_ratio=1.5, warmup_updates=2,
                              ema_decay=0.5, output_dir=scratch, sample_keys=("sample_index",))
        metrics = ScalarMetricCallback(every_n=2, sinks=[sink])
        group = CallbackGroup(config=None, trainer=None)
        group._callbacks.extend([monitor, metrics])
        trainer = Trainer(grad_accum_steps=2, callbacks=group, device=torch.device("cpu"))
        train = StatefulDataLoader(Rows(13, 71), batch_size=2, shuffle=True, seed=9, num_workers=0, pin_memory=False)
        held_out = StatefulDataLoader(Rows(6, 72), batch_size=2, shuffle=False, seed=9, num_workers=0,
                                      pin_memory=False)
        torch.manual_seed(8)
        done = trainer.train(model, train, held_out, grad_scaler=torch.amp.GradScaler(device="cpu", enabled=False),
                             max_iterations=7, validation_interval=3, max_val_steps=2, validate_at_start=True)
        out["loop/iterations"] = int(done)
        out["loop/spike_files"] = sorted(p.name for p in Path(scratch).rglob("*.json"))
        spikes = []
        for path in sorted(Path(scratch).rglob("*.json")):
            event = json.loads(path.read_text())
            spikes.append(sorted((k, v) for k, v in event.items() if k not in ("timestamp", "time", "host")))
        out["loop/spikes"] = repr(spikes)
    out["loop/metrics"] = sink.rows
    out["loop/cursor"] = sorted(train.state_dict().items())
    out["loop/lr"] = [float(group["lr"]) for group in optimizer.param_groups]
    for name, value in model.state_dict().items():
        out[f"loop/state/{name}"] = value


def _tiny_decoders(out: dict) -> None:
    import tempfile
    from pathlib import Path

    from wm.codecs import TAEW22SuperDecoder
    from wm.codecs._taehv.taehv import TAEHV, StreamingTAEHV

    def seeded(arch: str) -> TAEHV:
        model = TAEHV(None, arch_name=arch).float().eval()
        g = torch.Generator().manual_seed(81)
        with torch.no_grad():
            for name, tensor in sorted(model.state_dict().items()):
                if tensor.is_floating_point():
                    spread = (1.0 / max(1, tensor[0].numel())) ** 0.5 if tensor.ndim > 1 else 0.02
                    tensor.copy_(torch.randn(tensor.shape, generator=g) * spread)
        return model

    g = torch.Generator().manual_seed(82)
    latent = torch.randn(1, 3, 48, 4, 6, generator=g)           # N, T, C, H, W
    frames = torch.rand(1, 9, 3, 32, 48, generator=g)
    with torch.no_grad():
        for arch in ("taew2_2", "taew2_2_super"):
            model = seeded(arch)
            out[f"tiny/{arch}/keys"] = sorted(model.state_dict())
            out[f"tiny/{arch}/decode/parallel"] = model.decode_video(latent, parallel=True, show_progress_bar=False)
            out[f"tiny/{arch}/decode/sequential"] = model.decode_video(latent, parallel=False,
                                                                       show_progress_bar=False)
            if arch == "taew2_2":
                out["tiny/encode"] = model.encode_video(frames, parallel=True, show_progress_bar=False)
                out["tiny/encode/sequential"] = model.encode_video(frames, parallel=False, show_progress_bar=False)
                stream = StreamingTAEHV(model)
                pieces = []
                for index in range(latent.shape[1]):
                    piece = stream.decode(latent[:, index:index + 1])
                    while piece is not None:
                        pieces.append(piece)
                        piece = stream.decode()
                pieces.extend(stream.flush_decoder())
                out["tiny/stream"] = torch.cat(pieces, dim=1)
        with tempfile.TemporaryDirectory() as scratch:
            path = Path(scratch) / "taew2_2_super.pth"
            torch.save(seeded("taew2_2_super").state_dict(), path)
            decoder = TAEW22SuperDecoder(path)
            clip = latent.transpose(1, 2).contiguous()           # N, 48, T, H, W
            out["tiny/super/decode"] = decoder.decode(clip)
            running = decoder.stream("cpu")
            out["tiny/super/stream/0"] = running.decode(clip[:, :, :1])
            out["tiny/super/stream/1"] = running.decode(clip[:, :, 1:])
            running.reset()
            out["tiny/super/stream/again"] = running.decode(clip[:, :, :2])


def _streams(out: dict) -> None:
    import os

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_probe import batch_of, seeded_, tiny_config

    from wm.codecs import Wan22VAECodec
    from wm.models.flow import rf_interpolate
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network
    from wm.networks.cosmos3.network import Cosmos3Condition
    from wm.networks.cosmos3.reference import denoise_with_references
    from wm.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy

    config = tiny_config()
    net = build_network(config, init_device="cpu").float().eval()
    seeded_(net, 0)
    cond = Cosmos3Conditioner(config=config, codec=Wan22VAECodec(pretrained_path="unused", decoder=None),
                              geometry_noise_sigma=0.0, init_device="cpu", empty_prompt_ids=(3, 4, 5)).float()
    seeded_(cond.text_encoder, 1)
    batch = cond.encode(batch_of(13), training=False)
    condition = cond.condition(batch)
    other = cond.condition(cond.encode(batch_of(13, seed=4), training=False))
    latent = batch["latent"]
    noise = torch.randn(latent.shape, generator=torch.Generator().manual_seed(5))

    def part(source, lo: int, hi: int) -> Cosmos3Condition:
        return Cosmos3Condition(text=source.text, depth=source.depth[:, :, lo:hi],
                                normal=source.normal[:, :, lo:hi], fps=source.fps)

    with torch.no_grad():
        for rope in ("absolute", "contiguous", "top_aligned"):
            stream = Cosmos3Stream(net, StreamPolicy(block_frames=4, sink_frames=1, history_frames=4, rope=rope,
                                                     train_frames=13))
            stream.start(latent[:, :, :1], part(condition, 0, 1))
            for block in range(3):
                lo, hi = 1 + 4 * block, 5 + 4 * block
                noisy = rf_interpolate(latent[:, :, lo:hi], noise[:, :, lo:hi], torch.tensor([0.6]))
                if block == 2:
                    stream.update_text(other.text)                  # a new prompt mid-stream
                out[f"streams/{rope}/velocity/{block}"] = stream.denoise(noisy, torch.tensor([0.6]),
                                                                         part(condition, lo, hi))
                if block == 1 and rope == "top_aligned":
                    references = [latent[:, :, 9:10], latent[:, :, 12:13]]
                    out["streams/references"] = denoise_with_references(
                        stream, noisy, torch.tensor([0.6]), part(condition, lo, hi), references)
                    out["streams/no_references"] = denoise_with_references(
                        stream, noisy, torch.tensor([0.6]), part(condition, lo, hi), [])
                stream.commit(latent[:, :, lo:hi], part(condition, lo, hi))
            out[f"streams/{rope}/keys"] = torch.stack([key.clone() for key in stream.keys])
            out[f"streams/{rope}/values"] = torch.stack([value.clone() for value in stream.values])
            stream.reset()
            stream.start(latent[:, :, 1:2], part(condition, 1, 2))
            out[f"streams/{rope}/restart"] = stream.denoise(noise[:, :, 2:6], torch.tensor([0.9]),
                                                           part(condition, 2, 6))


def _sampling(out: dict) -> None:
    """``sample()`` of the three objectives on small towers, with a stand-in for the codec."""
    import os

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_probe import batch_of, seeded_, tiny_config

    from wm.codecs import Wan22VAECodec
    from wm.infra.parallel import ParallelConfig
    from wm.models.autoregressive import AutoregressiveModel
    from wm.models.diffusion import DiffusionModel
    from wm.models.dmd import DMDModel
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network

    def pixels(latent: torch.Tensor) -> torch.Tensor:
        """Stands in for the VAE decoder (no weights here): three latent channels as 'pixels'."""
        return (latent[:, :3] * 0.25).repeat_interleave(2, dim=-1)

    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)

    def conditioner():
        made = Cosmos3Conditioner(config=config, geometry_noise_sigma=0.0, init_device="cpu",
                                  empty_prompt_ids=(3, 4, 5),
                                  codec=Wan22VAECodec(pretrained_path="unused", decoder=None))
        made.codec.decode = pixels
        return made

    def finish(model):
        model.parallelize("cpu")
        seeded_(model.conditioner.text_encoder, 1)
        return model.eval()

    def record(label: str, panels) -> None:
        out[f"sampling/{label}/panels"] = sorted(panels)
        for name, value in panels.items():
            out[f"sampling/{label}/{name}"] = value

    def data_for(model, frames: int, seed: int):
        batch = batch_of(frames, seed=seed)
        batch["sample_id"] = torch.tensor([17])
        batch["depth_video"] = torch.rand(1, 3, frames, 4, 4, generator=torch.Generator().manual_seed(seed))
        return model.prepare_data_batch(batch)

    net = build_network(config, init_device="cpu")
    seeded_(net, 0)
    bidirectional = finish(DiffusionModel(net=net, conditioner=conditioner(), parallel=plain,
                                          conditioner_parallel=plain,
                                          sampling={"num_steps": 3, "guidance": 2.0, "seed": 4}))
    record("bidirectional", bidirectional.sample(data_for(bidirectional, 5, 11)))
    record("bidirectional/plain", bidirectional.sample(data_for(bidirectional, 5, 11), guidance=1.0, seed=9))
    try:
        bidirectional.sample(data_for(bidirectional, 5, 11), steps=3)
    except TypeError as error:
        out["sampling/unknown_option"] = str(error)
    for mode in ("teacher_forcing", "diffusion_forcing"):
        net = build_network(config, init_device="cpu")
        seeded_(net, 0)
        model = finish(AutoregressiveModel(net=net, conditioner=conditioner(), mode=mode, block_frames=4,
                                           parallel=plain, conditioner_parallel=plain))
        out[f"sampling/{mode}/defaults"] = sorted((k, repr(v)) for k, v in model.sampling.items())
        record(mode, model.sample(data_for(model, 9, 12), num_steps=2, guidance=1.5))
        record(f"{mode}/window", model.sample(data_for(model, 9, 12), num_steps=2, guidance=1.0, sink_blocks=0,
                                              recent_blocks=1))
    towers = [build_network(config, init_device="cpu") for _ in range(3)]
    for index, tower in enumerate(towers):
        seeded_(tower, 20 + index)
    distilled = finish(DMDModel(student=towers[0], real_score=towers[1], fake_score=towers[2],
                                conditioner=conditioner(), block_frames=4, student_parallel=plain,
                                score_parallel=plain, seed=3))
    out["sampling/dmd/defaults"] = sorted((k, repr(v)) for k, v in distilled.sampling.items())
    record("dmd", distilled.sample(data_for(distilled, 9, 13)))
    kept = distilled.checkpoint_model_state_dict(dict(distilled.state_dict()))
    out["sampling/dmd/saved_roles"] = sorted({key.split(".")[0] for key in kept})


def _conditioner_raw(out: dict) -> None:
    """Raw batches through the conditioner: pixels, captions with their suffix, the negative
    prompt, the geometry pipeline and its latent noise; the VAE encoder and the tokenizer are
    replaced by simple deterministic stand-ins (no weights, no vocabulary files here)."""
    import json
    import os
    import tempfile
    from pathlib import Path

    import transformers

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_probe import seeded_, tiny_config

    from wm.codecs import Wan22VAECodec
    from wm.networks.cosmos3 import Cosmos3Conditioner
    from wm.networks.cosmos3.geometry import GeometryAugmentationConfig

    class Characters:
        def apply_chat_template(self, messages, **options):
            assert options == {"tokenize": True, "add_generation_prompt": True, "add_vision_id": False,
                               "return_dict": False}, options
            return [3 + ord(c) % 120 for c in messages[0]["content"]]

    transformers.AutoTokenizer.from_pretrained = staticmethod(lambda *args, **kwargs: Characters())

    def encode(pixels: torch.Tensor) -> torch.Tensor:
        n, c, t, h, w = pixels.shape
        low = torch.nn.functional.adaptive_avg_pool3d(pixels.float(), (1 + (t - 1) // 4, h // 16, w // 16))
        return low.repeat(1, 16, 1, 1, 1).to(pixels.dtype)

    g = torch.Generator().manual_seed(91)
    raw = {
        "video": torch.randint(0, 256, (2, 5, 3, 64, 96), generator=g, dtype=torch.uint8),
        "depth": torch.rand(2, 5, 1, 64, 96, generator=g) * 20.0 + 0.5,
        "normal": torch.randint(0, 256, (2, 5, 3, 64, 96), generator=g, dtype=torch.uint8),
        "caption": ["  a red cube on a table ", "camera pans left."],
        "fps": torch.tensor([16.0, 24.0]), "sample_id": torch.tensor([5, 6]),
        "depth_scale": torch.tensor([1.0, 3.0]),
        "depth_scale_jitter_eligible": torch.tensor([True, False]),
        "depth_scale_jitter_bounds": torch.tensor([[0.5, 2.0], [0.5, 2.0]]),
    }
    augmentation = GeometryAugmentationConfig(
        modality_dropout_probability=0.3, spatial_probability=1.0, spatial_max_scale=1.1,
        spatial_max_shift_fraction=0.05, texture_suppression_probability=0.5, texture_downsample_min=1.5,
        texture_downsample_max=2.5)
    with tempfile.TemporaryDirectory() as scratch:
        negative = Path(scratch) / "negative.json"
        negative.write_text(json.dumps({"avoid": ["blur", "noise"], "style": "none."}))
        conditioner = Cosmos3Conditioner(
            config=tiny_config(), codec=Wan22VAECodec(pretrained_path="unused", decoder=None),
            geometry_augmentation=augmentation, geometry_noise_sigma=0.4, empty_prompt_ids=(3, 4, 5),
            tokenizer_path="unused", negative_prompt_path=str(negative), max_text_tokens=40, init_device="cpu")
        conditioner.codec.encode = encode
        seeded_(conditioner.text_encoder, 1)
        conditioner = conditioner.float()
        for training in (True, False):
            label = "train" if training else "eval"
            torch.manual_seed(13)
            encoded = conditioner.encode({key: (value.clone() if torch.is_tensor(value) else list(value))
                                          for key, value in raw.items()}, training=training)
            out[f"raw/{label}/keys"] = sorted(encoded)
            for key, value in encoded.items():
                if torch.is_tensor(value):
                    out[f"raw/{label}/{key}"] = value
            condition = conditioner.condition(encoded, drop=torch.tensor([False, True]))
            out[f"raw/{label}/depth"] = condition.depth
            out[f"raw/{label}/normal"] = condition.normal
            out[f"raw/{label}/text_valid"] = condition.text.valid_lengths
            out[f"raw/{label}/text_keys"] = torch.stack(list(condition.text.keys))
            if not training:
                unwanted = conditioner.condition(encoded, negative=True)
                out["raw/eval/negative_valid"] = unwanted.text.valid_lengths
                out["raw/eval/negative_keys"] = torch.stack(list(unwanted.text.keys))
                panels = conditioner.visuals(encoded)
                out["raw/eval/panels"] = sorted(panels)
                for name, value in panels.items():
                    out[f"raw/eval/panel/{name}"] = value


def _sampling_callback(out: dict) -> None:
    """Periodic sampling inside a training run: which batches are sampled and with which options,
    that sampling leaves the training random streams alone, and the files the media writer leaves
    (single-frame artifacts as PNG, so that no video encoder is involved)."""
    import hashlib
    import tempfile
    from pathlib import Path

    from wm.data.loader import StatefulDataLoader
    from wm.infra.callbacks import CallbackGroup, ImageVideoArtifactWriter, PeriodicSampleCallback
    from wm.infra.model import Model
    from wm.infra.trainer import Trainer

    calls = []

    class Toy(Model):
        def __init__(self) -> None:
            super().__init__()
            self.scale = torch.nn.Parameter(torch.tensor(0.5))

        def parallelize(self, device) -> None:
            return None

        def training_step(self, data_batch, iteration):
            noise = torch.rand(())                          # consumes the global stream
            loss = ((self.scale * data_batch["x"]).mean() - noise).square()
            return {"metrics/noise": noise}, loss

        def validation_step(self, data_batch, iteration):
            return self.training_step(data_batch, iteration)

        def sample(self, data_batch, **sampling_options):
            calls.append((bool(self.training), sorted((k, repr(v)) for k, v in sampling_options.items()),
                          data_batch["sample_index"].tolist()))
            torch.rand(3)                                   # must not disturb training
            base = data_batch["x"].reshape(-1, 1, 1, 1, 1).expand(-1, 3, 1, 6, 8) * 0.1
            ramp = torch.linspace(-1, 1, 8).view(1, 1, 1, 1, 8)
            return {"depth": base + ramp, "normal": base - ramp, "ground_truth": base * ramp,
                    "sample": (base + 0.3 * ramp).clamp(-1, 1), "comparison": base * 0.5}

    class Rows(torch.utils.data.Dataset):
        def __len__(self) -> int:
            return 8

        def __getitem__(self, index: int):
            return {"x": torch.tensor(float(index)), "sample_index": torch.tensor(index),
                    "validation_sample_seed": torch.tensor(100 + index)}

    model = Toy()
    optimizer = torch.optim.SGD(model.parameters(), lr=0.01)
    model.optimizer_dict = {"net": optimizer}
    model.scheduler_dict = {"net": torch.optim.lr_scheduler.LambdaLR(optimizer, lr_lambda=lambda step: 1.0)}
    with tempfile.TemporaryDirectory() as scratch:
        def writer():
            return ImageVideoArtifactWriter(image_format="png", grid_layout=["depth", "normal", "ground_truth", "sample"],
                                            grid_name="comparison", save_individual_artifacts=True)

        group = CallbackGroup(config=None, trainer=None)
        group._callbacks.extend([
            PeriodicSampleCallback(2, str(Path(scratch) / "held_out"), writer(), source="validation", max_batches=2,
                                   sampling_options={"steps": 4}),
            PeriodicSampleCallback(3, str(Path(scratch) / "seen"), writer(), source="train", seed_batch_key=None,
                                   sampling_options={"steps": 2})])
        trainer = Trainer(grad_accum_steps=1, callbacks=group, device=torch.device("cpu"))
        torch.manual_seed(21)
        trainer.train(model, StatefulDataLoader(Rows(), batch_size=2, shuffle=True, seed=1, num_workers=0,
                                                pin_memory=False),
                      StatefulDataLoader(Rows(), batch_size=2, shuffle=False, seed=1, num_workers=0, pin_memory=False),
                      grad_scaler=torch.amp.GradScaler(device="cpu", enabled=False), max_iterations=6,
                      validation_interval=2, max_val_steps=3, validate_at_start=True)
        files = sorted(str(p.relative_to(scratch)) for p in Path(scratch).rglob("*") if p.is_file())
        out["sampler/files"] = files
        out["sampler/digests"] = [hashlib.sha256((Path(scratch) / name).read_bytes()).hexdigest() for name in files]
        # the artifact rules on their own: refusals, name clashes, a grid whose panels are missing
        plain = ImageVideoArtifactWriter(image_format="png", grid_layout=["a", "b", "c"], grid_name="a",
                                         save_individual_artifacts=False)
        image = torch.zeros(2, 3, 1, 4, 4)
        for label, value in (("text", {"a": image, "note": "text"}), ("number", 3.0),
                             ("partial_grid", {"a": image, "b": image}), ("tensor", image),
                             ("unbatched", image[0]), ("images", image[:, :, 0]), ("gray", image[:, :1]),
                             ("integers", image.long()), ("two_dims", image[0, 0, 0]),
                             ("clash", {"a": image, "b": image + 0.5, "c": image - 0.5, "a/": image})):
            target = Path(scratch) / "rules" / label
            try:
                plain.write(value, output_dir=str(target), split="validation", iteration=1, rank=2)
                out[f"sampler/rules/{label}"] = sorted(p.name for p in target.rglob("*") if p.is_file())
            except Exception as error:
                out[f"sampler/rules/{label}"] = f"{type(error).__name__}: {error}"
    out["sampler/calls"] = calls
    out["sampler/scale"] = model.scale.detach().clone()
    out["sampler/next_random"] = torch.rand(2)


def _codec_surface(out: dict) -> None:
    """What the codec wrapper promises without weights: factors, frame arithmetic, the latent
    normalisation tables, the encoder window rule, refusals, and the hand-over to a tiny decoder."""
    from wm.codecs import Wan22VAECodec, wan22

    class Tiny:
        def decode(self, latent):
            return latent[:, :3] + 1.0

    codec = Wan22VAECodec("unused", dtype="float32", decoder=Tiny())
    out["codec/factors"] = [codec.spatial_compression_factor, codec.latent_channels,
                            codec.temporal_compression_factor, str(codec.dtype)]
    out["codec/latent_frames"] = [codec.latent_frames(n) for n in (1, 2, 5, 81, 93, 241)]
    out["codec/pixel_frames"] = [codec.pixel_frames(n) for n in (1, 2, 21, 61)]
    mean, inverse = codec._normalization(torch.device("cpu"))
    out["codec/mean"], out["codec/inverse_std"] = mean, inverse
    out["codec/tables"] = [tuple(wan22.WAN22_LATENTS_MEAN), tuple(wan22.WAN22_LATENTS_STD)]
    out["codec/window"] = [codec._encode_window(shape) for shape in ((240, 416), (256, 256), (480, 832),
                                                                     (640, 640), (720, 1280), (641, 2000))]
    out["codec/handed_over"] = codec.decode(torch.ones(1, 48, 2, 2, 2))
    for label, call in (("encode", lambda: codec.encode(torch.ones(1, 3, 1, 16, 16, dtype=torch.int32))),
                        ("decode", lambda: codec.decode(torch.ones(1, 48, 1, 2, 2, dtype=torch.int64)))):
        try:
            call()
        except Exception as error:
            out[f"codec/refusal/{label}"] = f"{type(error).__name__}: {error}"
    half = Wan22VAECodec("unused", device="cpu", temporal_compression_factor=8)
    out["codec/other"] = [str(half.dtype), half.latent_frames(17), half.pixel_frames(3),
                          str(half.preferred_device)]


def _model_base(out: dict) -> None:
    """The objective base class: trainable patterns over aliased parameters, parameter groups with
    the decay split, bindings of two roles with their refusals, cadence, and a two-closure step
    through the trainer (two roles updated in one step, gradients synchronised on the last)."""
    from wm.infra.callbacks import CallbackGroup
    from wm.infra.model import Model
    from wm.infra.trainer import Trainer

    class Twin(Model):
        def __init__(self, **options) -> None:
            super().__init__(**options)
            g = torch.Generator().manual_seed(3)
            self.left, self.right = torch.nn.Linear(4, 4), torch.nn.Linear(4, 4)
            self.tied = torch.nn.Linear(4, 4, bias=False)
            self.tied.weight = self.left.weight                 # one tensor, two names
            self.norm = torch.nn.LayerNorm(4)
            with torch.no_grad():
                for parameter in self.parameters():
                    parameter.copy_(torch.randn(parameter.shape, generator=g))
            self.active = ("a", "b")

        def parallelize(self, device) -> None:
            return None

        def get_optimizer_names(self, iteration):
            return self.active

        def training_step_closures(self, data_batch, iteration):
            yield "a", lambda: ({"metrics/a": torch.tensor(1.0)}, self.left(data_batch).square().mean()), False
            yield "b", lambda: ({"metrics/b": torch.tensor(2.0)}, self.right(data_batch).abs().mean()), True

        def sample(self, data_batch, **sampling_options):
            return None

    def live(model):
        return sorted(name for name, p in model.named_parameters(remove_duplicate=False) if p.requires_grad)

    model = Twin()
    model.configure_trainable_parameters([r"tied\.weight", r"norm\..*"])
    out["base/live/alias"] = live(model)
    model.configure_trainable_parameters(r"right\.(weight|bias)")
    out["base/live/string"] = live(model)
    model.configure_trainable_parameters(None)
    out["base/live/none"] = live(model)
    model.configure_trainable_parameters([r".*"], module=model.norm)
    out["base/live/module"] = live(model)
    model.requires_grad_(True)

    def shapes(groups):
        return [(sorted((k, repr(v)) for k, v in group.items() if k != "params"),
                 [tuple(p.shape) for p in group["params"]]) for group in groups]

    out["base/groups/plain"] = shapes(Twin()._group_trainable_parameters())
    out["base/groups/split"] = shapes(Twin(optimizer_split_decay_groups=True)._group_trainable_parameters())
    declared = Twin(optimizer_parameter_groups=[
        {"patterns": [r"tied\.weight"], "lr": 0.5}, {"patterns": r".*bias", "weight_decay": 0.0},
        {"patterns": r"nothing", "lr": 9.0}], optimizer_split_decay_groups=True)
    out["base/groups/declared"] = shapes(declared._group_trainable_parameters())
    out["base/cadence"] = [bool(model.is_cadence_due(i, n)) for i in (0, 1, 4, 8) for n in (None, 0, 4)]

    first = torch.optim.SGD([model.left.weight, model.left.bias], lr=0.1)
    second = torch.optim.SGD([model.right.weight, model.right.bias], lr=0.2)
    constant = lambda step: 1.0   # noqa: E731
    model.optimizer_dict = {"a": first, "b": second}
    model.scheduler_dict = {"a": torch.optim.lr_scheduler.LambdaLR(first, constant),
                            "b": torch.optim.lr_scheduler.LambdaLR(second, constant)}
    out["base/bindings"] = [binding.name for binding in model.get_optimizer_bindings(0)]

    def refusal(label):
        try:
            model.get_optimizer_bindings(0)
            out[f"base/refusal/{label}"] = "accepted"
        except Exception as error:
            out[f"base/refusal/{label}"] = f"{type(error).__name__}: {error}"

    model.active = ()
    refusal("none")
    model.active = ("a", "a")
    refusal("twice")
    model.active = ("a", "c")
    refusal("unknown")
    model.active = ("a", "b")
    model.scheduler_dict["b"] = torch.optim.lr_scheduler.LambdaLR(first, constant)
    refusal("foreign_scheduler")
    overlapping = torch.optim.SGD([model.left.weight, model.right.bias], lr=0.1)
    model.optimizer_dict["b"] = overlapping
    model.scheduler_dict["b"] = torch.optim.lr_scheduler.LambdaLR(overlapping, constant)
    refusal("shared_parameter")
    model.optimizer_dict["b"] = second
    model.scheduler_dict["b"] = torch.optim.lr_scheduler.LambdaLR(second, constant)

    trainer = Trainer(grad_accum_steps=2, callbacks=CallbackGroup(config=None, trainer=None),
                      device=torch.device("cpu"))
    scaler = torch.amp.GradScaler(device="cpu", enabled=False)
    g = torch.Generator().manual_seed(4)
    steps = []
    for micro in range(4):
        result = trainer.training_step(model, scaler, torch.randn(3, 4, generator=g), iteration=micro // 2,
                                       grad_accum_step=micro % 2)
        steps.append((float(result.loss), result.grad_accum_step, bool(result.did_update),
                      sorted(result.output_batch)))
    out["base/steps"] = steps
    for name, value in model.state_dict().items():
        out[f"base/state/{name}"] = value
    try:
        trainer.training_step(model, scaler, torch.randn(3, 4, generator=g), iteration=3, grad_accum_step=2)
    except Exception as error:
        out["base/refusal/accum_step"] = f"{type(error).__name__}: {error}"


def _history_windows(out: dict) -> None:
    """Block-causal passes under a bounded history (sink + recent blocks), in both forcing modes,
    and the cached rollout under the same window; ``forward`` with several known frames and
    feature taps."""
    import os

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_probe import batch_of, seeded_, tiny_config

    from wm.codecs import Wan22VAECodec
    from wm.models.flow import rf_interpolate
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network
    from wm.protocols import HistoryWindow

    config = tiny_config()
    net = build_network(config, init_device="cpu").float().eval()
    seeded_(net, 0)
    cond = Cosmos3Conditioner(config=config, codec=Wan22VAECodec(pretrained_path="unused", decoder=None),
                              geometry_noise_sigma=0.0, init_device="cpu", empty_prompt_ids=(3, 4, 5)).float()
    seeded_(cond.text_encoder, 1)
    batch = cond.encode(batch_of(13), training=False)
    condition = cond.condition(batch)
    latent = batch["latent"]
    noise = torch.randn(latent.shape, generator=torch.Generator().manual_seed(5))
    sigma = torch.tensor([[0.9] * 4 + [0.5] * 4 + [0.2] * 4])
    targets = rf_interpolate(latent[:, :, 1:], noise[:, :, 1:], sigma)
    with torch.no_grad():
        for label, window in (("sink1_recent1", HistoryWindow(sink_blocks=1, recent_blocks=1)),
                              ("recent1", HistoryWindow(sink_blocks=0, recent_blocks=1)),
                              ("everything", HistoryWindow())):
            out[f"window/{label}/diffusion"] = net.forward_ar(latent[:, :, :1], targets, sigma, condition,
                                                              block_frames=4, history=window)
            out[f"window/{label}/teacher"] = net.forward_ar(latent[:, :, :1], targets, sigma, condition,
                                                            block_frames=4, clean=latent[:, :, 1:], history=window)
            cache = net.prefill(latent[:, :, :1], condition, history=window)
            for block in range(3):
                lo, hi = 4 * block, 4 * block + 4
                out[f"window/{label}/cached/{block}"] = net.denoise(cache, targets[:, :, lo:hi],
                                                                    sigma[:, lo])
                cache = net.commit(cache, latent[:, :, 1 + lo:1 + hi])
        flat = rf_interpolate(latent, noise, torch.tensor([0.6]))
        flat[:, :, :3] = latent[:, :, :3]
        out["window/known3"] = net(flat, torch.tensor([0.6]), condition, known_frames=3)


def _initializations(out: dict) -> None:
    """``train.model_initializations``: overlays from a released-weights directory (safetensors,
    source prefix and key patterns, one or several destinations, the resume subset) and from a
    checkpoint written by the same tree, applied to a model with several roles; the plan they are
    coalesced into; refusals for keys that do not fit."""
    import tempfile
    import warnings
    from pathlib import Path

    from safetensors.torch import save_file

    from wm.infra.checkpoint import DistributedCheckpointer
    from wm.infra.checkpoint.plan import plan_model_initializations
    from wm.infra.model import Model

    class Tower(torch.nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.layers = torch.nn.ModuleList(torch.nn.Linear(3, 3) for _ in range(2))
            self.head = torch.nn.Linear(3, 2)

    class Roles(Model):
        def __init__(self) -> None:
            super().__init__()
            self.student, self.fake, self.frozen = Tower(), Tower(), Tower()
            with torch.no_grad():
                for parameter in self.parameters():
                    parameter.fill_(-1.0)

        def parallelize(self, device) -> None:
            return None

        def sample(self, data_batch, **sampling_options):
            return None

    g = torch.Generator().manual_seed(77)
    released = {f"net.{name}": torch.randn(value.shape, generator=g) for name, value in Tower().state_dict().items()}
    released["net.unrelated.weight"] = torch.zeros(2)
    entries = {
        "layers_student": {"path": "RELEASED", "model_key_prefix": "student", "source_model_key_prefix": "net",
                           "source_model_key_patterns": [r"layers\..*"]},
        "layers_fake": {"path": "RELEASED", "model_key_prefix": "fake", "source_model_key_prefix": "net",
                        "source_model_key_patterns": [r"layers\..*"]},
        "frozen": {"path": "RELEASED", "model_key_prefixes": ["frozen"], "source_model_key_prefix": "net",
                   "source_model_key_patterns": [r"layers\..*", r"head\..*"],
                   "resume_model_key_prefixes": ["frozen"]},
        "skipped": {"path": None, "model_key_prefix": "student"},
    }
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for resume in (False, True):
            plan = plan_model_initializations(entries, resume=resume)
            out[f"init/plan/{resume}"] = [sorted((k, repr(v)) for k, v in item.load_kwargs().items()) for item in plan]
        with tempfile.TemporaryDirectory() as scratch:
            directory = Path(scratch) / "released"
            directory.mkdir()
            save_file(released, str(directory / "model.safetensors"))
            located = {label: {**entry, "path": None if entry["path"] is None else str(directory)}
                       for label, entry in entries.items()}
            saver = DistributedCheckpointer(Path(scratch) / "checkpoints")
            for resume in (False, True):
                model = Roles()
                saver.initialize_model(model, located, resume=resume)
                for name, value in model.state_dict().items():
                    out[f"init/{'resume' if resume else 'fresh'}/{name}"] = value
            # a checkpoint of this tree as the source of another role
            model = Roles()
            saver.initialize_model(model, located, resume=False)
            optimizer = torch.optim.SGD(model.parameters(), lr=0.1)
            scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, lambda step: 1.0)
            saver.save(model, {"net": optimizer}, {"net": scheduler}, None, iteration=3)
            saver.finalize()
            out["init/latest"] = (Path(scratch) / "checkpoints" / "latest").read_text()
            other = Roles()
            saver.initialize_model(other, {"from_run": {
                "path": str(Path(scratch) / "checkpoints" / "iter_000000003"), "model_key_prefix": "fake",
                "source_model_key_prefix": "student"}}, resume=False)
            for name, value in other.state_dict().items():
                out[f"init/from_run/{name}"] = value
            try:
                saver.initialize_model(Roles(), {"bad": {"path": str(directory), "model_key_prefix": "student",
                                                          "source_model_key_prefix": "missing"}}, resume=False)
                out["init/refusal"] = "accepted"
            except Exception as error:
                out["init/refusal"] = type(error).__name__


def _fused_adam(out: dict) -> None:
    """The optimizer on the CPU path: Adam and AdamW, without first or second moment, FP32 master
    weights under bf16 parameters, per-group options, bias correction off, a state dict that is
    saved and loaded back; construction refusals."""
    from wm.infra.optim import FusedAdam

    def parameters(dtype):
        g = torch.Generator().manual_seed(15)
        made = [torch.nn.Parameter(torch.randn(shape, generator=g).to(dtype)) for shape in ((5, 3), (3,), (2, 2, 2))]
        return made, g

    variants = {
        "adamw": dict(lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1, adam_w_mode=True),
        "adam_l2": dict(lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1, adam_w_mode=False),
        "no_first_moment": dict(lr=2e-3, betas=(0.0, 0.999), eps=1e-8),
        "no_second_moment": dict(lr=2e-3, betas=(0.9, 0.0), eps=1e-3),
        "no_bias_correction": dict(lr=1e-2, betas=(0.8, 0.9), eps=1e-6, bias_correction=False),
        "master": dict(lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01, use_te_capturable_kernel=True,
                       master_weights=True),
    }
    for label, options in variants.items():
        dtype = torch.bfloat16 if label == "master" else torch.float32
        made, g = parameters(dtype)
        groups = [{"params": made[:2]}, {"params": made[2:], "lr": options["lr"] * 0.5, "weight_decay": 0.0}]
        optimizer = FusedAdam(groups, **options)
        for step in range(4):
            for parameter in made:
                parameter.grad = torch.randn(parameter.shape, generator=g).to(dtype) * (1.0 + step)
            optimizer.step()
            if step == 1:
                saved = optimizer.state_dict()
                optimizer.load_state_dict(saved)        # the state survives its own round trip
        for index, parameter in enumerate(made):
            out[f"adam/{label}/parameter/{index}"] = parameter.detach().float()
        state = optimizer.state_dict()["state"]
        out[f"adam/{label}/state_fields"] = [sorted(state[index]) for index in sorted(state)]
        for index in sorted(state):
            for field, value in sorted(state[index].items()):
                if torch.is_tensor(value):
                    out[f"adam/{label}/state/{index}/{field}"] = value.detach().float().reshape(-1)
                    out[f"adam/{label}/state_dtype/{index}/{field}"] = str(value.dtype)
    made, _ = parameters(torch.float32)
    for label, options in (("amsgrad", dict(amsgrad=True)), ("master_without_kernel", dict(master_weights=True)),
                           ("negative_lr", dict(lr=-1.0)), ("beta_one", dict(betas=(1.0, 0.9))),
                           ("three_betas", dict(betas=(0.9, 0.9, 0.9)))):
        try:
            FusedAdam(made, **options)
            out[f"adam/refusal/{label}"] = "accepted"
        except Exception as error:
            out[f"adam/refusal/{label}"] = f"{type(error).__name__}: {error}"


def _constants(out: dict) -> None:
    """Tables and defaults that users and checkpoints depend on: key patterns of the released
    weights, LoRA module lists, the empty prompt, configuration defaults, the distillation
    endpoints, and the building blocks of the recipes."""
    import dataclasses

    from wm.models import dmd
    from wm.networks import cosmos3
    from wm.networks.cosmos3.geometry import GeometryAugmentationConfig
    from wm.networks.cosmos3.streaming import StreamPolicy

    def plain(value):
        if dataclasses.is_dataclass(value) and not isinstance(value, type):
            return sorted((f.name, repr(getattr(value, f.name))) for f in dataclasses.fields(value))
        if isinstance(value, dict):
            return sorted((str(k), repr(v)) for k, v in value.items())
        if isinstance(value, (list, tuple, set, frozenset)):
            return [repr(v) for v in value]
        return repr(value)

    for name in ("TEXT_ENCODER_KEYS", "GEN_KEYS", "LORA_ATTENTION_MODULES", "LORA_MLP_MODULES"):
        if hasattr(cosmos3, name):
            out[f"constants/cosmos3/{name}"] = plain(getattr(cosmos3, name))
    out["constants/cosmos3/names"] = sorted(n for n in dir(cosmos3) if n.isupper() and not n.startswith("_"))
    out["constants/config"] = plain(cosmos3.Cosmos3Config())
    out["constants/stream_policy"] = plain(StreamPolicy())
    out["constants/geometry"] = plain(GeometryAugmentationConfig())
    out["constants/dmd/endpoints"] = plain(dmd.RCM_ENDPOINTS)
    out["constants/dmd/gan"] = plain(dmd.GANConfig())
    from wm.networks.cosmos3 import conditioner

    out["constants/empty_prompt"] = plain(conditioner.COSMOS3_EMPTY_PROMPT_IDS)
    try:
        from wm.configs.experiments import cosmos3 as recipes

        for name in ("GEOMETRY_AUGMENTATION", "LORA_TRAINABLE", "RELEASED_TRANSFORMER"):
            out[f"constants/recipes/{name}"] = plain(getattr(recipes, name))
    except Exception as error:
        out["constants/recipes"] = f"{type(error).__name__}: {error}"


def _recipes(out: dict) -> None:
    """The configuration tree of every recipe before resolution (targets, constants, callbacks,
    optimizer and scheduler settings, initialisations), flattened to ``path = value`` lines with
    the package root of ``_target_`` strings normalised."""
    import importlib
    from collections.abc import Mapping

    def flatten(node, prefix, lines):
        if isinstance(node, Mapping) or (hasattr(node, "items") and hasattr(node, "keys")):
            for key in node.keys():
                try:
                    child = node._get_node(key)._value() if False else dict.__getitem__(node, key)
                except Exception:
                    try:
                        child = node.get(key) if not hasattr(node, "_raw") else node._raw(key)
                    except Exception:
                        child = "<unreadable>"
                flatten(child, f"{prefix}.{key}" if prefix else str(key), lines)
        elif isinstance(node, (list, tuple)) or type(node).__name__ in ("ListConfig", "LazyList"):
            for index, child in enumerate(list(node)):
                flatten(child, f"{prefix}[{index}]", lines)
        else:
            text = repr(node) if not isinstance(node, str) else node
            if isinstance(node, str):
                for root in ("agentgarten_b200.", "wm."):
                    if text.startswith(root):
                        text = "<package>." + text[len(root):]
            lines.append(f"{prefix} = {text}")

    for name in ("bidirectional", "ar_teacher_forcing", "ar_diffusion_forcing", "dmd", "dmd_gan", "dmd_gan_exact",
                 "dmd_gan_lora"):
        try:
            module = importlib.import_module(f"wm.configs.experiments.cosmos3.{name}")
            lines: list[str] = []
            flatten(module.build_config(), "", lines)
            out[f"recipes/{name}"] = sorted(lines)
        except Exception as error:
            out[f"recipes/{name}"] = f"{type(error).__name__}: {error}"


def _utilities(out: dict) -> None:
    """Tree mapping of tensors, seeding, the mode / gradient-flag guards, atomic file helpers,
    image encoding and the random-state capture of a single process."""
    import collections
    import random
    import tempfile
    from pathlib import Path

    import numpy as np

    from wm.infra import io
    from wm.infra.rng_state import (capture_distributed_rng_state, isolated_rng, restore_distributed_rng_state,
                                    validate_distributed_rng_state)
    from wm.infra.utils import frozen_parameters, map_tensors, preserve_training_mode, set_random_seed, to

    Pair = collections.namedtuple("Pair", "left right")
    shared = torch.arange(4.0)
    tree = {"a": shared, "b": [shared, Pair(torch.ones(2), "text")], "c": collections.defaultdict(list, {"k": shared}),
            "d": (1, 2.5, None, b"bytes", range(3)), "e": collections.OrderedDict(z=torch.zeros(1))}
    mapped = map_tensors(tree, lambda tensor: tensor * 2)
    out["util/map/types"] = [type(mapped).__name__, type(mapped["b"]).__name__, type(mapped["b"][1]).__name__,
                             type(mapped["c"]).__name__, type(mapped["d"]).__name__, type(mapped["e"]).__name__,
                             repr(mapped["d"]), repr(mapped["c"].default_factory)]
    out["util/map/shared"] = [mapped["a"] is mapped["b"][0], mapped["a"] is mapped["c"]["k"]]
    out["util/map/values"] = torch.cat([mapped["a"], mapped["b"][1].left, mapped["e"]["z"]])
    moved = to({"x": torch.zeros(2, 3, 4, 5), "y": torch.ones(2, dtype=torch.int64)}, device="cpu",
               dtype=torch.float64, memory_format=torch.channels_last)
    out["util/to"] = [str(moved["x"].dtype), str(moved["y"].dtype),
                      bool(moved["x"].is_contiguous(memory_format=torch.channels_last))]
    set_random_seed(1234)
    out["util/seeded"] = [random.random(), float(np.random.rand()), float(torch.rand(()))]
    module = torch.nn.Sequential(torch.nn.Linear(2, 2), torch.nn.Dropout(0.5))
    module[1].eval()
    module[0].weight.requires_grad_(False)
    with preserve_training_mode(module), frozen_parameters(module):
        module.eval()
        inside = [p.requires_grad for p in module.parameters()]
    out["util/guards"] = [inside, [p.requires_grad for p in module.parameters()],
                          [m.training for m in module.modules()]]
    with tempfile.TemporaryDirectory() as scratch:
        target = io.join_path(scratch, "deep", "file.txt")
        io.atomic_put_text("héllo\n", target)
        io.atomic_put(b"\x00\x01", io.join_path(scratch, "deep", "file.bin"))
        out["util/io"] = [io.exists(target), io.get_text(target), io.get(io.join_path(scratch, "deep", "file.bin")),
                          io.exists(io.join_path(scratch, "missing")),
                          sorted(p.name for p in (Path(scratch) / "deep").iterdir())]
    pixels = (np.arange(6 * 8 * 3) % 251).astype(np.uint8).reshape(6, 8, 3)
    out["util/png"] = io.encode_image(pixels, file_format="png").getvalue()
    out["util/jpg"] = io.encode_image(pixels, file_format="jpg", quality=80).getvalue()
    set_random_seed(77)
    state = capture_distributed_rng_state()
    validate_distributed_rng_state(state)
    out["util/rng/keys"] = sorted(state)
    first = [random.random(), float(np.random.rand()), float(torch.rand(()))]
    with isolated_rng():
        random.random(), np.random.rand(), torch.rand(3)
    second = [random.random(), float(np.random.rand()), float(torch.rand(()))]
    restore_distributed_rng_state(state)
    again = [random.random(), float(np.random.rand()), float(torch.rand(()))]
    out["util/rng/draws"] = [first, second, again]
    try:
        validate_distributed_rng_state({"rank_00000001": {}})
        out["util/rng/refusal"] = "accepted"
    except Exception as error:
        out["util/rng/refusal"] = type(error).__name__


def _runtime_misc(out: dict) -> None:
    """Gradient clipping helpers (groups, an unlimited norm, non-finite gradients, shared
    parameters), lazy calls and their instantiation rules, rank helpers without a process group,
    and the metric callback's handling of odd step outputs and of a failing sink."""
    import fractions

    from wm.infra import distributed
    from wm.infra.callbacks import ScalarMetricCallback
    from wm.infra.callbacks.grad_clip import clip_grad_norm_, clip_grad_norm_groups_
    from wm.infra.config import LazyCall, instantiate

    def parameters(values):
        made = []
        for value in values:
            parameter = torch.nn.Parameter(torch.zeros(len(value)))
            parameter.grad = torch.tensor(value)
            made.append(parameter)
        return made

    a, b, c = parameters([[3.0, 4.0], [12.0], [0.0, 0.0]])
    frozen = torch.nn.Parameter(torch.zeros(1), requires_grad=False)
    bare = torch.nn.Parameter(torch.zeros(1))
    total, roles = clip_grad_norm_groups_({"first": [a, frozen, bare], "second": [b, a, c]}, 6.5)
    out["clip/total"], out["clip/roles"] = total, sorted((k, float(v)) for k, v in roles.items())
    out["clip/grads"] = torch.cat([a.grad, b.grad, c.grad])
    a, b = parameters([[3.0, 4.0], [12.0]])
    out["clip/observe"] = clip_grad_norm_([a, b], float("inf"))
    out["clip/observe/grads"] = torch.cat([a.grad, b.grad])
    a, b = parameters([[float("nan"), 1.0], [2.0]])
    out["clip/nonfinite"] = clip_grad_norm_([a, b], 1.0)
    out["clip/nonfinite/grads"] = torch.cat([a.grad, b.grad])
    out["clip/nothing"] = repr(clip_grad_norm_groups_({"x": [frozen, bare]}, 1.0))
    for label, bound in (("negative", -1.0), ("nan", float("nan"))):
        try:
            clip_grad_norm_([a], bound)
            out[f"clip/refusal/{label}"] = "accepted"
        except Exception as error:
            out[f"clip/refusal/{label}"] = f"{type(error).__name__}: {error}"

    lazy = LazyCall(fractions.Fraction)(numerator=3, denominator=4)
    out["lazy/keys"] = sorted(str(k) for k in lazy)
    out["lazy/target"] = lazy["_target_"]
    out["lazy/value"] = str(instantiate(lazy))
    out["lazy/override"] = str(instantiate(lazy, denominator=5))
    nested = {"_target_": "builtins.dict", "inner": LazyCall(fractions.Fraction)(numerator=1, denominator=2),
              "plain": [1, {"_target_": "builtins.int", "_recursive_": True}]}
    built = instantiate(nested)
    out["lazy/nested"] = [type(built).__name__, str(built["inner"]), repr(list(built["plain"]))]
    kept = instantiate({"_target_": "builtins.dict", "_recursive_": False,
                        "inner": {"_target_": "builtins.int"}})
    out["lazy/not_recursive"] = repr(dict(kept["inner"]))
    out["lazy/passthrough"] = [repr(instantiate(3)), repr(instantiate([1, "x"])), repr(instantiate({"k": (1, 2)}))]
    for label, config in (("missing_module", {"_target_": "no_such_package.thing"}),
                          ("missing_name", {"_target_": "builtins.no_such_name"}),
                          ("not_a_string", {"_target_": 3}), ("not_callable", {"_target_": "math.pi"})):
        try:
            instantiate(config)
            out[f"lazy/refusal/{label}"] = "accepted"
        except Exception as error:
            out[f"lazy/refusal/{label}"] = type(error).__name__
    try:
        LazyCall(3)
    except Exception as error:
        out["lazy/refusal/target"] = type(error).__name__

    out["ranks"] = [distributed.get_rank(), distributed.get_world_size(), distributed.get_local_rank(),
                    distributed.get_local_world_size(), bool(distributed.is_rank0())]

    class Sink:
        def __init__(self, broken: bool) -> None:
            self.broken, self.rows = broken, []

        def write(self, metrics, *, iteration):
            if self.broken:
                raise OSError("disk full")
            self.rows.append((int(iteration), sorted((k, round(float(v), 6)) for k, v in metrics.items())))

    good, bad = Sink(False), Sink(True)
    callback = ScalarMetricCallback(every_n=2, sinks=[bad, None, good])
    model = torch.nn.Linear(1, 1)
    for iteration in range(1, 5):
        outputs = {"metrics/ok": torch.tensor(float(iteration)), "metrics/nan": torch.tensor(float("nan")),
                   "metrics/vector": torch.ones(2), "metrics/text": "skip", "metrics/number": 2.0 * iteration,
                   "other": torch.tensor(9.0)}
        callback.on_training_step_batch_end(model, {}, outputs, torch.tensor(0.5 * iteration), iteration=iteration - 1)
        callback.on_training_step_end(model, {}, outputs, torch.tensor(0.5 * iteration), iteration=iteration)
    out["metrics/rows"] = good.rows
    out["metrics/sinks_left"] = len([sink for sink in callback.sinks])


def _resume_rules(out: dict) -> None:
    """Resume under a changed recipe: the current learning rates, schedule and optimizer options
    win, progress (update counts, moments) is restored, parameters that had no optimizer state get
    none, selected components only, and the iteration and data cursor come back."""
    import tempfile
    import warnings
    from pathlib import Path

    from wm.data.loader import StatefulDataLoader
    from wm.infra.checkpoint import DistributedCheckpointer
    from wm.infra.model import Model
    from wm.infra.optim import FusedAdam, LinearWarmup

    class Toy(Model):
        def __init__(self, seed: int) -> None:
            super().__init__()
            g = torch.Generator().manual_seed(seed)
            self.used, self.unused = torch.nn.Linear(3, 3), torch.nn.Linear(3, 1)
            with torch.no_grad():
                for parameter in self.parameters():
                    parameter.copy_(torch.randn(parameter.shape, generator=g))

        def parallelize(self, device) -> None:
            return None

        def sample(self, data_batch, **sampling_options):
            return None

    class Rows(torch.utils.data.Dataset):
        def __len__(self) -> int:
            return 10

        def __getitem__(self, index: int):
            return {"index": torch.tensor(index)}

    def job(seed: int, lr: float, warmup: int, betas):
        model = Toy(seed)
        optimizer = FusedAdam(model.parameters(), lr=lr, betas=betas, eps=1e-8, weight_decay=0.0)
        scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, LinearWarmup(warmup_steps=warmup, start_factor=0.5))
        loader = StatefulDataLoader(Rows(), batch_size=2, shuffle=True, seed=4, num_workers=0, pin_memory=False)
        return model, optimizer, scheduler, loader

    def steps(model, optimizer, scheduler, count: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        for _ in range(count):
            optimizer.zero_grad(set_to_none=True)
            model.used(torch.randn(4, 3, generator=g)).square().mean().backward()   # `unused` gets no gradient
            optimizer.step()
            scheduler.step()

    with warnings.catch_warnings(), tempfile.TemporaryDirectory() as scratch:
        warnings.simplefilter("ignore")
        model, optimizer, scheduler, loader = job(1, 0.01, 4, (0.9, 0.99))
        steps(model, optimizer, scheduler, 3, 50)
        iterator = iter(loader)
        next(iterator), next(iterator)
        saver = DistributedCheckpointer(Path(scratch) / "checkpoints")
        saver.save(model, {"net": optimizer}, {"net": scheduler}, None, iteration=3, dataloader=loader,
                   runtime_metadata={"note": "first run"})
        saver.finalize()
        out["resume/files"] = sorted(str(p.relative_to(scratch)) for p in Path(scratch).rglob("*")
                                     if p.is_file() and "tensor" not in p.parts)

        fresh, new_optimizer, new_scheduler, new_loader = job(2, 0.02, 8, (0.8, 0.95))
        result = DistributedCheckpointer(Path(scratch) / "checkpoints").load(
            fresh, {"net": new_optimizer}, {"net": new_scheduler}, None, path="latest", dataloader=new_loader,
            runtime_metadata={"note": "second run"})
        out["resume/iteration"] = int(result.iteration)
        out["resume/cursor"] = sorted(new_loader.state_dict().items())
        group = new_optimizer.param_groups[0]
        out["resume/options"] = [float(group["lr"]), tuple(float(b) for b in group["betas"]), float(group["initial_lr"])]
        out["resume/schedule"] = [int(new_scheduler.last_epoch), [float(v) for v in new_scheduler.get_last_lr()]]
        state = new_optimizer.state_dict()["state"]
        out["resume/state_of"] = sorted(state)
        for index in sorted(state):
            for name, value in sorted(state[index].items()):
                if torch.is_tensor(value):
                    out[f"resume/state/{index}/{name}"] = value.detach().float().reshape(-1)
        for name, value in fresh.state_dict().items():
            out[f"resume/model/{name}"] = value
        steps(fresh, new_optimizer, new_scheduler, 2, 51)
        for name, value in fresh.state_dict().items():
            out[f"resume/continued/{name}"] = value
        out["resume/continued_lr"] = [float(v) for v in new_scheduler.get_last_lr()]

        only_model, other_optimizer, other_scheduler, _ = job(3, 0.05, 2, (0.9, 0.99))
        result = DistributedCheckpointer(Path(scratch) / "checkpoints").load(
            only_model, {"net": other_optimizer}, {"net": other_scheduler}, None, path="latest",
            components=("model",))
        out["resume/model_only"] = [int(result.iteration), len(other_optimizer.state_dict()["state"]),
                                    int(other_scheduler.last_epoch)]
        out["resume/model_only/weight"] = only_model.used.weight.detach().clone()
        nothing = DistributedCheckpointer(Path(scratch) / "checkpoints").load(
            Toy(4), {}, {}, None, path=None)
        out["resume/nothing"] = int(nothing.iteration)
        try:
            DistributedCheckpointer(Path(scratch) / "elsewhere").load(Toy(4), {}, {}, None, path="latest")
            out["resume/no_pointer"] = "accepted"
        except Exception as error:
            out["resume/no_pointer"] = type(error).__name__


def _batched_network(out: dict) -> None:
    """Two samples with prompts of different lengths and different frame rates through the text
    tower and the generation tower (bidirectional and block-causal), feature taps, patch helpers."""
    import os

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_probe import seeded_, tiny_config

    from wm.codecs import Wan22VAECodec
    from wm.models.flow import rf_interpolate
    from wm.networks.cosmos3 import Cosmos3Conditioner, build_network
    from wm.networks.cosmos3 import network as network_module

    config = tiny_config()
    net = build_network(config, init_device="cpu").float().eval()
    seeded_(net, 0)
    cond = Cosmos3Conditioner(config=config, codec=Wan22VAECodec(pretrained_path="unused", decoder=None),
                              geometry_noise_sigma=0.0, init_device="cpu", empty_prompt_ids=(3, 4, 5)).float()
    seeded_(cond.text_encoder, 1)
    g = torch.Generator().manual_seed(61)
    shape = (2, 48, 5, 8, 8)
    ids = torch.randint(3, 128, (2, 14), generator=g)
    mask = torch.ones(2, 14, dtype=torch.bool)
    mask[1, 6:] = False
    batch = {"latent": torch.randn(shape, generator=g), "depth_latent": torch.randn(shape, generator=g),
             "normal_latent": torch.randn(shape, generator=g), "text_input_ids": ids,
             "text_attention_mask": mask, "fps": torch.tensor([16.0, 30.0])}
    encoded = cond.encode(batch, training=False)
    with torch.no_grad():
        condition = cond.condition(encoded)
        out["batched/text_valid"] = condition.text.valid_lengths
        out["batched/text_keys"] = torch.stack(list(condition.text.keys))
        out["batched/text_values"] = torch.stack(list(condition.text.values))
        dropped = cond.condition(encoded, drop=torch.tensor([True, False]))
        out["batched/dropped_valid"] = dropped.text.valid_lengths
        latent = encoded["latent"]
        noise = torch.randn(latent.shape, generator=g)
        sigma = torch.tensor([0.7, 0.2])
        noisy = rf_interpolate(latent, noise, sigma)
        noisy[:, :, :1] = latent[:, :, :1]
        out["batched/forward"] = net(noisy, sigma, condition, known_frames=1)
        block_sigma = torch.tensor([[0.9] * 4, [0.4] * 4])
        targets = rf_interpolate(latent[:, :, 1:], noise[:, :, 1:], block_sigma)
        out["batched/forward_ar"] = net.forward_ar(latent[:, :, :1], targets, block_sigma, condition, block_frames=4)
        import dataclasses

        scaled = build_network(dataclasses.replace(config, timestep_scale=0.7), init_device="cpu").float().eval()
        seeded_(scaled, 0)
        out["batched/timestep_scale"] = scaled.embed_rgb(latent[:1, :, :3], torch.tensor([[0.123, 0.456, 0.789]]))
        patches = network_module.patchify(latent[:, :, :2], config.patch_size)
        out["batched/patchify"] = patches
        out["batched/unpatchify"] = network_module.unpatchify(patches, channels=48, grid=(4, 4),
                                                               patch_size=config.patch_size)


def _skipped_update(out: dict) -> None:
    """An update whose gradients are not finite: nothing steps, the schedule does not move, the
    gradients are cleared, the hooks fire in the documented order, and the next update goes
    through; with the monitor attached the event is recorded and the norm is reported."""
    import tempfile

    from wm.infra.callbacks import Callback, CallbackGroup, GradClipMonitor
    from wm.infra.model import Model
    from wm.infra.trainer import Trainer

    class Toy(Model):
        def __init__(self) -> None:
            super().__init__()
            self.weight = torch.nn.Parameter(torch.tensor([1.0, -2.0, 0.5]))

        def parallelize(self, device) -> None:
            return None

        def training_step(self, data_batch, iteration):
            loss = (self.weight * data_batch["x"]).sum()
            return {"metrics/plain": loss.detach()}, loss

        def sample(self, data_batch, **sampling_options):
            return None

    class Recorder(Callback):
        def __init__(self) -> None:
            super().__init__()
            self.events = []

        def on_training_step_start(self, model, data_batch, iteration=0):
            self.events.append(("start", iteration))

        def on_before_optimizer_step(self, model_ddp, optimizer, scheduler, grad_scaler, iteration=0):
            self.events.append(("before_step", iteration))

        def on_optimizer_step_skipped(self, model_ddp, optimizer_names, iteration=0):
            self.events.append(("skipped", tuple(optimizer_names), iteration))

        def on_after_optimizer_step(self, model_ddp, optimizer_name, optimizer, scheduler, iteration=0):
            self.events.append(("after_step", optimizer_name, iteration))

        def on_before_zero_grad(self, model_ddp, optimizer, scheduler, iteration=0):
            self.events.append(("before_zero_grad", iteration))

        def on_training_step_batch_end(self, model, data_batch, output_batch, loss, iteration=0):
            self.events.append(("batch_end", iteration, sorted(output_batch)))

        def on_training_step_end(self, model, data_batch, output_batch, loss, iteration=0):
            self.events.append(("step_end", iteration))

    with tempfile.TemporaryDirectory() as scratch:
        model, recorder = Toy(), Recorder()
        monitor = GradClipMonitor(max_norm=10.0, spike_threshold=None, spike_ratio=None, output_dir=scratch)
        optimizer = torch.optim.SGD(model.parameters(), lr=0.1)
        scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, lambda step: 1.0 / (1 + step))
        model.optimizer_dict, model.scheduler_dict = {"net": optimizer}, {"net": scheduler}
        group = CallbackGroup(config=None, trainer=None)
        group._callbacks.extend([monitor, recorder])
        trainer = Trainer(grad_accum_steps=1, callbacks=group, device=torch.device("cpu"))
        scaler = torch.amp.GradScaler(device="cpu", enabled=False)
        rows = []
        for iteration, batch in enumerate((torch.tensor([1.0, 2.0, 3.0]), torch.tensor([1.0, float("inf"), 3.0]),
                                           torch.tensor([0.5, 0.5, 0.5]))):
            result = trainer.training_step(model, scaler, {"x": batch}, iteration=iteration)
            rows.append((bool(result.did_update), bool(result.found_nonfinite), result.grad_accum_step,
                         sorted(result.output_batch), model.weight.grad is None, int(scheduler.last_epoch),
                         [round(float(v), 6) for v in model.weight.detach()]))
        out["skip/rows"] = rows
        out["skip/events"] = recorder.events
        out["skip/reported"] = sorted((k, round(float(v), 6)) for k, v in result.output_batch.items()
                                      if k.startswith("metrics/"))


def _refusals(out: dict) -> None:
    """What the constructors and entry points refuse, and in which words."""
    from wm.data.loader import StatefulDataLoader
    from wm.infra.callbacks import GradClip, PeriodicSampleCallback
    from wm.infra.optim import CosineDecay, LinearWarmup, LinearWarmupCosineDecay
    from wm.infra.trainer import Trainer
    from wm.models.dmd import GANConfig, PhaseClock
    from wm.models.flow import FlowUniPC, RectifiedFlowSchedule, UniformShift
    from wm.networks.cosmos3.geometry import GeometryAugmentationConfig
    from wm.networks.cosmos3.streaming import StreamPolicy
    from wm.networks.discriminator import DiscriminatorHead
    from wm.protocols import HistoryWindow

    cases = {
        "policy/block": lambda: StreamPolicy(block_frames=0),
        "policy/sink": lambda: StreamPolicy(sink_frames=-1),
        "policy/history": lambda: StreamPolicy(block_frames=4, sink_frames=5, history_frames=6),
        "policy/rope": lambda: StreamPolicy(rope="sideways"),
        "policy/train_frames": lambda: StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, train_frames=4),
        "window/negative": lambda: HistoryWindow(sink_blocks=-1),
        "clock/zero": lambda: PhaseClock(fake_score_updates_per_student=0),
        "gan/kind": lambda: GANConfig(regularization="imaginary"),
        "gan/weight": lambda: GANConfig(regularization_weight=-1.0),
        "schedule/shift": lambda: RectifiedFlowSchedule(shift=0.0),
        "schedule/kind": lambda: RectifiedFlowSchedule(train_distribution="triangular"),
        "uniform/shift": lambda: UniformShift(float("nan")),
        "geometry/probability": lambda: GeometryAugmentationConfig(spatial_probability=1.5),
        "geometry/scale": lambda: GeometryAugmentationConfig(spatial_max_scale=0.5),
        "geometry/range": lambda: GeometryAugmentationConfig(texture_downsample_min=2.0, texture_downsample_max=1.0),
        "geometry/selection": lambda: GeometryAugmentationConfig(modality_selection="neither"),
        "head/layers": lambda: DiscriminatorHead(hidden_size=8, feature_layers=(1, 1), num_heads=2),
        "head/heads": lambda: DiscriminatorHead(hidden_size=10, feature_layers=(1,), num_heads=4),
        "head/sign": lambda: DiscriminatorHead(hidden_size=8, feature_layers=(1,), num_heads=2, initial_logit_sign=0.5),
        "lr/cosine": lambda: CosineDecay(decay_steps=0),
        "lr/min_factor": lambda: CosineDecay(decay_steps=10, min_factor=1.5),
        "lr/both": lambda: LinearWarmupCosineDecay(warmup_steps=10, decay_steps=5),
        "lr/warmup": lambda: LinearWarmup(warmup_steps=10, start_factor=-0.1),
        "clip/bound": lambda: GradClip(max_norm=-1.0),
        "trainer/accum": lambda: Trainer(grad_accum_steps=0),
        "sampler/source": lambda: PeriodicSampleCallback(1, "out", None, source="test"),
        "sampler/batches": lambda: PeriodicSampleCallback(1, "out", None, max_batches=-1),
        "loader/cursor": lambda: StatefulDataLoader([1, 2, 3], batch_size=1, num_workers=0, pin_memory=False
                                                    ).load_state_dict({"epoch": -1, "batch_offset": 0}),
        "solver/steps": lambda: FlowUniPC(0, shift=1.0).run(torch.zeros(1), lambda x, s: x),
    }
    for label, make in cases.items():
        try:
            made = make()
            out[f"refusal/{label}"] = f"accepted: {type(made).__name__}"
        except Exception as error:
            out[f"refusal/{label}"] = f"{type(error).__name__}: {error}"


def _vae(out: dict) -> None:
    from wm.codecs import wan22

    small = dict(dim=16, dec_dim=16, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=1)
    if hasattr(wan22, "_Wan22VAE"):
        vae = wan22._Wan22VAE(temperal_downsample=(False, True, True), **small)
    else:
        vae = wan22.Wan22VAE(temporal_downsample=(False, True, True), **small)
    vae = vae.float().eval()
    g = torch.Generator().manual_seed(51)
    with torch.no_grad():
        for name, tensor in sorted(vae.state_dict().items()):
            if not tensor.is_floating_point():
                continue
            if name.endswith("gamma"):
                tensor.copy_(1.0 + 0.1 * torch.randn(tensor.shape, generator=g))
            elif tensor.ndim > 1:
                tensor.copy_(torch.randn(tensor.shape, generator=g) * (1.0 / max(1, tensor[0].numel())) ** 0.5)
            else:
                tensor.copy_(torch.randn(tensor.shape, generator=g) * 0.02)
    out["vae/keys"] = sorted(vae.state_dict())
    clip = torch.rand(1, 3, 9, 32, 32, generator=g) * 2.0 - 1.0
    scale = (torch.linspace(-0.2, 0.2, 4), torch.linspace(0.8, 1.2, 4))
    with torch.no_grad():
        latent = vae.encode(clip, scale, temporal_window=4)
        out["vae/latent"] = latent
        out["vae/latent/window8"] = vae.encode(clip, scale, temporal_window=8)
        out["vae/pixels"] = vae.decode(latent, scale)
        out["vae/single_frame"] = vae.encode(clip[:, :, :1], (0.0, 1.0), temporal_window=4)


def artifact_exchange(save_to: str, load_from: str | None = None) -> dict:
    """Export a small seeded student + text tower with ``save_artifact``; when ``load_from`` names
    an export (of either tree), inspect and load it and return what came out."""
    import os
    from pathlib import Path

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_probe import seeded_, tiny_config

    from wm.inference.cosmos3 import (Cosmos3Artifact, Cosmos3ArtifactSpec, inspect_artifact, load_artifact,
                                      save_artifact)
    from wm.networks.cosmos3 import build_network
    from wm.networks.cosmos3.network import Cosmos3TextEncoder

    config = tiny_config()
    lora = {"rank": 4, "alpha": 8.0, "dropout": 0.0, "target_modules": ["to_q", "to_out"]}
    student = build_network(config, init_device="cpu", lora=lora).float()
    text = Cosmos3TextEncoder(config).float()
    seeded_(student, 30)
    seeded_(text, 31)
    spec = Cosmos3ArtifactSpec(checkpoint=Path(save_to), config=config, student=(), text=(),
                               tokenizer_path=Path(save_to) / "tokenizer", prompt_pixel_frames=13, iteration=42,
                               lora=lora)
    root = save_artifact(Cosmos3Artifact(student, text, spec), save_to)
    out: dict = {"saved/files": sorted(p.name for p in Path(root).iterdir()),
                 "saved/student_keys": sorted(student.state_dict()), "saved/text_keys": sorted(text.state_dict())}
    if load_from is not None:
        found = inspect_artifact(load_from)
        out["loaded/iteration"] = found.iteration
        out["loaded/frames"] = found.prompt_pixel_frames
        out["loaded/lora"] = sorted((k, repr(v)) for k, v in dict(found.lora).items())
        out["loaded/tokenizer"] = Path(found.tokenizer_path).name
        out["loaded/config"] = sorted((k, repr(v)) for k, v in vars(found.config).items()) \
            if hasattr(found.config, "__dict__") else repr(found.config)
        loaded = load_artifact(found, device="cpu", dtype=torch.float32)
        out["loaded/report"] = sorted((k, repr(v)) for k, v in loaded.report.items()
                                      if k not in ("checkpoint_path", "und_checkpoint_path", "implementation"))
        for name, value in loaded.student.state_dict().items():
            out[f"loaded/student/{name}"] = value
        for name, value in loaded.context_encoder.state_dict().items():
            out[f"loaded/text/{name}"] = value
    return out


def ddp_exchange() -> dict:
    """Run under a two-rank Gloo launch: loss closures through the data-parallel wrapper with two
    micro-batches per update.  Gradients stay local after the first micro-batch and are averaged
    over the ranks by the last backward pass; every rank ends with the same parameters."""
    import torch.distributed as dist

    from wm.infra import distributed
    from wm.infra.callbacks import CallbackGroup
    from wm.infra.model import Model
    from wm.infra.trainer import Trainer

    distributed.init(device="cpu", backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()

    class Toy(Model):
        def __init__(self) -> None:
            super().__init__()
            g = torch.Generator().manual_seed(3)
            self.body = torch.nn.Linear(3, 2)
            with torch.no_grad():
                for parameter in self.parameters():
                    parameter.copy_(torch.randn(parameter.shape, generator=g))

        def parallelize(self, device) -> None:
            return None

        def training_step(self, data_batch, iteration):
            loss = (self.body(data_batch["x"]) - data_batch["y"]).square().mean()
            return {"metrics/mse": loss.detach()}, loss

        def sample(self, data_batch, **sampling_options):
            return None

    model = Toy()
    wrapped = distributed.wrap_ddp(model, device="cpu")
    optimizer = torch.optim.SGD(model.parameters(), lr=0.1)
    model.optimizer_dict = {"net": optimizer}
    model.scheduler_dict = {"net": torch.optim.lr_scheduler.LambdaLR(optimizer, lambda step: 1.0)}
    trainer = Trainer(grad_accum_steps=2, callbacks=CallbackGroup(config=None, trainer=None),
                      device=torch.device("cpu"))
    scaler = torch.amp.GradScaler(device="cpu", enabled=False)
    g = torch.Generator().manual_seed(100 + rank)
    record: dict = {"wrapped": type(wrapped).__name__, "root": type(getattr(wrapped, "training_model", None)).__name__}
    for micro in range(4):
        batch = {"x": torch.randn(5, 3, generator=g), "y": torch.randn(5, 2, generator=g)}
        result = trainer.training_step(wrapped, scaler, batch, iteration=micro // 2, grad_accum_step=micro % 2)
        gradient = None if model.body.weight.grad is None else model.body.weight.grad.clone()
        gathered: list = [None] * world
        dist.all_gather_object(gathered, {"loss": float(result.loss), "updated": bool(result.did_update),
                                          "gradient": gradient, "weight": model.body.weight.detach().clone()})
        record[f"micro/{micro}"] = gathered
    dist.barrier()
    out: dict = {"ddp/wrapped": record["wrapped"], "ddp/root": record["root"]}
    for micro in range(4):
        rows = record[f"micro/{micro}"]
        out[f"ddp/{micro}/losses"] = [row["loss"] for row in rows]
        out[f"ddp/{micro}/updated"] = [row["updated"] for row in rows]
        out[f"ddp/{micro}/weights"] = torch.stack([row["weight"] for row in rows])
        if rows[0]["gradient"] is not None:
            out[f"ddp/{micro}/gradients"] = torch.stack([row["gradient"] for row in rows])
    distributed.destroy_process_group()
    return out if rank == 0 else {}


def transport_exchange() -> dict:
    """Run under a four-rank Gloo launch with context-parallel groups of two: micro-batch ``i`` is
    read and prepared by group member ``i % 2`` and handed to the other one together with the
    owner's random state; an early end and a failing dataset reach every rank."""
    import random

    import numpy as np
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    from wm.infra import distributed
    from wm.infra.batch_transport import fetch_batch, prepare_batch
    from wm.infra.model import ContextParallelContext

    distributed.init(device="cpu", backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mesh = init_device_mesh("cpu", (world // 2, 2), mesh_dim_names=("dp", "cp"))
    context = ContextParallelContext(mesh["cp"])
    record: dict = {"context": [context.size, context.rank, context.leader_global_rank, context.artifact_rank,
                                [list(group) for group in context.groups], bool(context.is_leader),
                                context.checkpoint_topology()]}

    def batches():
        for index in range(3):
            yield {"x": torch.full((2, 3), float(10 * rank + index)), "ids": [rank, index],
                   "nested": {"y": torch.arange(4) + rank, "name": f"clip-{rank}-{index}"}}

    def prepare(batch):
        # consumes the owner's random streams: the others must continue from the same point
        batch = dict(batch)
        batch["noise"] = torch.rand(2) + random.random() + float(np.random.rand())
        return batch

    random.seed(100 + rank)
    np.random.seed(200 + rank)
    torch.manual_seed(300 + rank)
    iterator = batches()
    steps = []
    for index in range(4):
        batch, exhausted, owner = fetch_batch(context, iterator, sequence_index=index)
        if exhausted:
            steps.append("end")
            break
        shared = prepare_batch(context, batch, owner_rank=owner, prepare=prepare)
        steps.append({"owner": owner, "x": shared["x"], "ids": shared["ids"], "y": shared["nested"]["y"],
                      "name": shared["nested"]["name"], "noise": shared["noise"],
                      "after": [random.random(), float(np.random.rand()), float(torch.rand(()))]})
    record["steps"] = steps

    def failing():
        yield {"x": torch.zeros(1)}
        if rank == 3:
            raise ValueError("corrupt sample")
        yield {"x": torch.zeros(1)}

    iterator = failing()
    fetch_batch(context, iterator, sequence_index=1)      # member 1 of every group reads its first item
    try:
        fetch_batch(context, iterator, sequence_index=3)  # and its second: rank 3 fails
        record["failure"] = "none"
    except RuntimeError as error:
        record["failure"] = ("rank 3" in str(error), "corrupt sample" in str(error))
    gathered: list = [None] * world
    dist.all_gather_object(gathered, record)
    dist.barrier()
    distributed.destroy_process_group()
    if rank != 0:
        return {}
    out: dict = {}
    for member, seen in enumerate(gathered):
        out[f"transport/{member}/context"] = repr(seen["context"])
        out[f"transport/{member}/failure"] = repr(seen["failure"])
        out[f"transport/{member}/steps"] = len(seen["steps"])
        for index, step in enumerate(seen["steps"]):
            if step == "end":
                out[f"transport/{member}/{index}"] = "end"
                continue
            out[f"transport/{member}/{index}/meta"] = repr((step["owner"], step["ids"], step["name"], step["after"]))
            out[f"transport/{member}/{index}/tensors"] = torch.cat([step["x"].reshape(-1), step["y"].float(),
                                                                    step["noise"]])
    return out


def run_exchange(save_to: str, load_from: str | None = None) -> dict:
    """Lay out a small training run (checkpoint of a bidirectional model, its resolved
    configuration, the released text tower it was initialised from) under ``save_to``; when
    ``load_from`` names such a run (of either tree), inspect its checkpoint and load it for
    serving."""
    import dataclasses
    import os
    from pathlib import Path

    import yaml
    from safetensors.torch import save_file

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from reference_probe import seeded_, tiny_config

    from wm.codecs import Wan22VAECodec
    from wm.inference.cosmos3 import inspect_artifact, load_artifact
    from wm.infra.checkpoint import DistributedCheckpointer
    from wm.infra.parallel import ParallelConfig
    from wm.models.diffusion import DiffusionModel
    from wm.networks.cosmos3 import TEXT_ENCODER_KEYS, Cosmos3Conditioner, build_network

    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)
    model = DiffusionModel(net=build_network(config, init_device="cpu"),
                           conditioner=Cosmos3Conditioner(config=config, geometry_noise_sigma=0.0, init_device="cpu",
                                                          empty_prompt_ids=(3, 4, 5),
                                                          codec=Wan22VAECodec(pretrained_path="unused", decoder=None)),
                           parallel=plain, conditioner_parallel=plain)
    model.parallelize("cpu")
    seeded_(model.net, 40)
    seeded_(model.conditioner.text_encoder, 41)
    run = Path(save_to)
    released = run / "released" / "transformer"
    released.mkdir(parents=True, exist_ok=True)
    save_file({key: value.detach().clone() for key, value in model.conditioner.text_encoder.state_dict().items()},
              str(released / "model.safetensors"))
    optimizer = torch.optim.SGD([p for p in model.net.parameters() if p.requires_grad], lr=0.1)
    scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, lambda step: 1.0)
    saver = DistributedCheckpointer(run / "checkpoints")
    saver.save(model, {"net": optimizer}, {"net": scheduler}, None, iteration=5)
    saver.finalize()
    topology = {f.name: getattr(config, f.name) for f in dataclasses.fields(config)}
    topology = {k: (list(v) if isinstance(v, tuple) else v) for k, v in topology.items()}
    resolved = {
        "model": {"net": {"config": topology, "lora": None},
                  "conditioner": {"tokenizer_path": "released/tokenizer"}},
        "dataloader_val": {"dataset": {"num_frames": 9}},
        "train": {"model_initializations": {"text": {
            "path": "released/transformer", "model_key_prefix": "conditioner.text_encoder",
            "source_model_key_prefix": "", "source_model_key_patterns": list(TEXT_ENCODER_KEYS)}}},
    }
    (run / "config.yaml").write_text(yaml.safe_dump(resolved))
    out: dict = {"run/files": sorted(str(p.relative_to(run)) for p in run.rglob("*")
                                     if p.is_file() and "tensor" not in p.parts)}
    if load_from is not None:
        source = Path(load_from)
        spec = inspect_artifact(source / "checkpoints" / "iter_000000005")
        out["run/spec"] = [spec.iteration, spec.prompt_pixel_frames, repr(spec.lora),
                           [(Path(s.path).name, s.prefix, tuple(s.patterns)) for s in spec.student],
                           [(Path(s.path).name, s.prefix, len(s.patterns)) for s in spec.text],
                           Path(spec.tokenizer_path).name]
        seen = []
        artifact = load_artifact(spec, device="cpu", dtype=torch.float32,
                                 progress=lambda label, done, total: seen.append((label, done, total)))
        out["run/progress"] = seen
        for name, value in artifact.student.state_dict().items():
            out[f"run/student/{name}"] = value
        for name, value in artifact.context_encoder.state_dict().items():
            out[f"run/text/{name}"] = value
        out["run/frozen"] = not any(p.requires_grad for p in artifact.student.parameters())
    return out


SECTIONS = {"flow": _flow, "lr": _lr, "geometry": _geometry, "media": _media, "policies": _policies,
            "seeded_modules": _seeded_modules, "data": _data, "training_loop": _training_loop,
            "tiny_decoders": _tiny_decoders, "streams": _streams, "sampling": _sampling, "conditioner_raw": _conditioner_raw,
            "sampling_callback": _sampling_callback, "codec_surface": _codec_surface, "model_base": _model_base,
            "history_windows": _history_windows, "initializations": _initializations, "fused_adam": _fused_adam, "constants": _constants, "recipes": _recipes, "utilities": _utilities, "runtime_misc": _runtime_misc, "resume_rules": _resume_rules, "batched_network": _batched_network, "skipped_update": _skipped_update, "refusals": _refusals,
            "vae": _vae}


def collect(sections=None) -> dict:
    out: dict = {}
    for name, section in SECTIONS.items():
        if sections and name not in sections:
            continue
        try:
            section(out)
        except Exception as error:   # recorded, so that the comparison names the section
            out[f"{name}/error"] = f"{type(error).__name__}: {error}"
    return out


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2] == "artifact":   # <out> artifact <save_to> [<load_from>]
        torch.save(artifact_exchange(*sys.argv[3:5]), sys.argv[1])
    elif len(sys.argv) > 2 and sys.argv[2] == "run":          # <out> run <save_to> [<load_from>]
        torch.save(run_exchange(*sys.argv[3:5]), sys.argv[1])
    elif len(sys.argv) > 2 and sys.argv[2] == "transport":   # under a four-rank launch; rank 0 writes
        found = transport_exchange()
        if found:
            torch.save(found, sys.argv[1])
    elif len(sys.argv) > 2 and sys.argv[2] == "ddp":      # under a two-rank launch; rank 0 writes
        found = ddp_exchange()
        if found:
            torch.save(found, sys.argv[1])
    else:
        torch.save(collect(sys.argv[2:] or None), sys.argv[1])
