"""Outputs of the package's pure and seeded functions, for differential tests.

The same file runs against either tree: with ``PYTHONPATH=baseline/_ref:baseline/shims`` the
imports below resolve to the unmodified reference package, inside this repository they resolve
to the ``wm`` alias of this package.  ``collect()`` returns ``{name: tensor | number | list}``;
as a script it writes that dictionary with ``torch.save``.  Every section is independent: a
section that cannot run in one tree records ``"<section>/error"`` instead of stopping the rest.

Covered: rectified-flow utilities and the UniPC solver, learning-rate factors, geometry
preprocessing and its seeded augmentations, media conversion and file names, the history window,
the phase clock of the distillation recipe, the stream position policy, seeded initialisation of
the discriminator head and of LoRA adapters, and the Wan 2.2 VAE (encode / decode of a small clip
with shared random weights).
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


SECTIONS = {"flow": _flow, "lr": _lr, "geometry": _geometry, "media": _media, "policies": _policies,
            "seeded_modules": _seeded_modules, "vae": _vae}


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
    torch.save(collect(sys.argv[2:] or None), sys.argv[1])
