"""Parity with the UNMODIFIED reference package on the CPU.

The reference runs in a child process whose import path holds only ``baseline/_ref`` and the
stand-ins of ``baseline/shims`` (``baseline/reference_probe.py``); this process loads the
state dicts it wrote into this package's modules and compares outputs, loss sequences and
updated parameters.
"""

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REFERENCE = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REFERENCE / "wm" / "__init__.py").exists(),
                                reason="the reference package is not installed under baseline/_ref")


def reference_env():
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    env["PYTHONPATH"] = os.pathsep.join((str(REFERENCE), str(ROOT / "baseline" / "shims")))
    return env


def probe(mode: str, path: Path, *extra: str):
    done = subprocess.run([sys.executable, str(ROOT / "baseline" / "reference_probe.py"), mode, str(path),
                           *extra], capture_output=True, text=True, timeout=900, env=reference_env(),
                          cwd=str(ROOT / "baseline"))
    assert done.returncode == 0, done.stderr[-3000:]
    return torch.load(path, weights_only=False)


def tiny_config():
    from agentgarten_b200.networks.cosmos3 import Cosmos3Config

    return Cosmos3Config(hidden_size=256, intermediate_size=1024, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=128,
                         mrope_section=(12, 10, 10), text_bucket_tokens=16,
                         special_tokens={"eos_token_id": 1, "start_of_generation": 2})


def batch_of(frames: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    shape = (1, 48, frames, 8, 8)
    return {"latent": torch.randn(shape, generator=g), "depth_latent": torch.randn(shape, generator=g),
            "normal_latent": torch.randn(shape, generator=g),
            "text_input_ids": torch.randint(3, 128, (1, 10), generator=g), "fps": torch.full((1,), 16.0)}


def test_network_outputs_equal_the_reference(tmp_path):
    """forward, forward_ar (both forcing modes), the cached rollout and a bounded stream with
    eviction give the reference's outputs from the reference's state dict."""
    from agentgarten_b200.models.flow import rf_interpolate
    from agentgarten_b200.networks.cosmos3 import build_network
    from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
    from agentgarten_b200.networks.cosmos3.network import Cosmos3Condition
    from agentgarten_b200.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy

    golden = probe("network", tmp_path / "network.pt")
    config = tiny_config()
    net = build_network(config, init_device="cpu").float().eval()
    net.load_state_dict(golden["net"], strict=True)
    cond = Cosmos3Conditioner(config=config, codec=None, geometry_noise_sigma=0.0, init_device="cpu",
                              empty_prompt_ids=(3, 4, 5)).float()
    cond.text_encoder.load_state_dict(golden["text_encoder"], strict=True)
    batch = cond.encode(golden["batch"], training=False)
    condition = cond.condition(batch)
    latent, noise = batch["latent"], golden["noise"]
    tol = dict(atol=1e-5, rtol=1e-5)
    with torch.no_grad():
        sigma = torch.tensor([0.7])
        noisy = rf_interpolate(latent, noise, sigma)
        noisy[:, :, :1] = latent[:, :, :1]
        assert torch.allclose(net(noisy, sigma, condition, known_frames=1), golden["forward"], **tol)
        block_sigma = golden["block_sigma"]
        targets = rf_interpolate(latent[:, :, 1:], noise[:, :, 1:], block_sigma)
        out = net.forward_ar(latent[:, :, :1], targets, block_sigma, condition, block_frames=4)
        assert torch.allclose(out, golden["forward_ar"], **tol)
        out = net.forward_ar(latent[:, :, :1], targets, block_sigma, condition, block_frames=4,
                             clean=latent[:, :, 1:])
        assert torch.allclose(out, golden["forward_ar_teacher"], **tol)
        cache = net.prefill(latent[:, :, :1], condition)
        first = net.denoise(cache, targets[:, :, :4], torch.tensor([0.9]))
        cache = net.commit(cache, latent[:, :, 1:5])
        second = net.denoise(cache, targets[:, :, 4:], torch.tensor([0.3]))
        assert torch.allclose(first, golden["cached"][0], **tol)
        assert torch.allclose(second, golden["cached"][1], **tol)

        def part(lo, hi):
            return Cosmos3Condition(text=condition.text, depth=condition.depth[:, :, lo:hi],
                                    normal=condition.normal[:, :, lo:hi], fps=condition.fps)

        stream = Cosmos3Stream(net, StreamPolicy(block_frames=4, sink_frames=1, history_frames=4,
                                                 rope="top_aligned", train_frames=9))
        stream.start(latent[:, :, :1], part(0, 1))
        for block in range(2):
            lo, hi = 1 + 4 * block, 5 + 4 * block
            got = stream.denoise(targets[:, :, lo - 1:hi - 1], torch.tensor([0.6]), part(lo, hi))
            assert torch.allclose(got, golden["streamed"][block], **tol)
            stream.commit(latent[:, :, lo:hi], part(lo, hi))
        for mine, theirs in zip(stream.keys, golden["stream_keys"], strict=True):
            assert torch.allclose(mine, theirs, **tol)  # evicted and re-rotated history


def test_seeded_training_repeats_the_reference_loss_sequence(tmp_path):
    """Five optimizer updates (two microbatches each, text dropout, gradient clipping, AdamW with
    FP32 masters, warm-up schedule) through this package's Trainer give the reference's losses
    and parameters."""
    from agentgarten_b200.infra.callbacks import CallbackGroup, GradClip
    from agentgarten_b200.infra.config import LazyCall
    from agentgarten_b200.infra.optim import FusedAdam, LinearWarmup
    from agentgarten_b200.infra.trainer import Trainer
    from agentgarten_b200.models.diffusion import DiffusionModel
    from agentgarten_b200.networks.cosmos3 import build_network
    from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
    from agentgarten_b200.parallel.engine import ParallelConfig

    golden = probe("train", tmp_path / "train.pt", "--steps", "5")
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        from reference_probe import seeded_
    finally:
        sys.path.pop(0)
    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)
    model = DiffusionModel(
        net=build_network(config, init_device="cpu"),
        conditioner=Cosmos3Conditioner(config=config, codec=None, geometry_noise_sigma=0.0,
                                       init_device="cpu", empty_prompt_ids=(3, 4, 5)),
        text_dropout=0.1, parallel=plain, conditioner_parallel=plain)
    model.parallelize("cpu")
    seeded_(model.net, 0)
    seeded_(model.conditioner.text_encoder, 1)
    model.train()
    optimizer = FusedAdam(model._group_trainable_parameters(), lr=1e-3, betas=(0.9, 0.99), eps=1e-8,
                          weight_decay=0.01, adam_w_mode=True, use_te_capturable_kernel=True,
                          master_weights=True)
    scheduler = torch.optim.lr_scheduler.LambdaLR(
        optimizer, lr_lambda=LinearWarmup(warmup_steps=4, start_factor=0.1))
    model.optimizer_dict, model.scheduler_dict = {"net": optimizer}, {"net": scheduler}
    callbacks = CallbackGroup(
        {"trainer": {"callbacks": {"grad_clip": LazyCall(GradClip)(max_norm=1.0)}}}, trainer=None)
    trainer = Trainer(grad_accum_steps=2, callbacks=callbacks, device=torch.device("cpu"))
    scaler = torch.amp.GradScaler(device="cpu", enabled=False)
    torch.manual_seed(1234)
    losses = []
    for step in range(5):
        for micro in range(2):
            data = model.prepare_data_batch(batch_of(5, seed=10 * step + micro))
            result = trainer.training_step(model, scaler, data, iteration=step, grad_accum_step=micro)
            losses.append(float(result.loss))
    assert losses == pytest.approx(golden["losses"], rel=2e-5, abs=2e-6)
    assert optimizer.param_groups[0]["lr"] == pytest.approx(golden["lr"])
    mine = model.net.state_dict()
    for name, theirs in golden["net"].items():
        assert torch.allclose(mine[name], theirs, atol=2e-5, rtol=1e-4), name


def test_autoregressive_objective_equals_the_reference(tmp_path):
    """Seeded training loss (text dropout, per-block sigmas, degraded clean history), gradient
    norm and validation loss of both forcing modes, and the history degradation itself."""
    from agentgarten_b200.models.autoregressive import AutoregressiveModel, corrupt_history
    from agentgarten_b200.networks.cosmos3 import build_network
    from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
    from agentgarten_b200.parallel.engine import ParallelConfig

    golden = probe("autoregressive", tmp_path / "ar.pt")
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        from reference_probe import seeded_
    finally:
        sys.path.pop(0)
    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)
    for mode in ("teacher_forcing", "diffusion_forcing"):
        model = AutoregressiveModel(
            net=build_network(config, init_device="cpu"),
            conditioner=Cosmos3Conditioner(config=config, codec=None, geometry_noise_sigma=0.0,
                                           init_device="cpu", empty_prompt_ids=(3, 4, 5)),
            mode=mode, block_frames=4, text_dropout=0.5, parallel=plain, conditioner_parallel=plain)
        model.parallelize("cpu")
        seeded_(model.net, 0)
        seeded_(model.conditioner.text_encoder, 1)
        model.train()
        data = model.prepare_data_batch(batch_of(9, seed=3))
        torch.manual_seed(77)
        report, loss = model.training_step(data, 0)
        loss.backward()
        norm = torch.sqrt(sum(p.grad.square().sum() for p in model.net.parameters() if p.grad is not None))
        model.eval()
        _, validation = model.validation_step(model.prepare_data_batch(batch_of(9, seed=4)), 0)
        want = golden[mode]
        assert float(loss) == pytest.approx(want["loss"], rel=2e-5), mode
        assert torch.allclose(report["sigma"], want["sigma"])
        assert float(norm) == pytest.approx(want["grad_norm"], rel=1e-4), mode
        assert float(validation) == pytest.approx(want["validation"], rel=2e-5), mode
    mine = corrupt_history(golden["frames"], torch.Generator().manual_seed(6))
    assert torch.allclose(mine, golden["corrupted"], atol=1e-6)


def test_adversarial_forcing_equals_the_reference(tmp_path):
    """Discriminator warm-up, student and fake-score iterations of the distillation objective on
    small towers: losses, per-role gradient norms and every reported scalar equal the
    reference's, with finite-difference and with exact R1/R2; so does the validation loss."""
    from agentgarten_b200.models.dmd import DMDModel, GANConfig
    from agentgarten_b200.networks.cosmos3 import build_network
    from agentgarten_b200.networks.cosmos3.conditioner import Cosmos3Conditioner
    from agentgarten_b200.networks.discriminator import DiscriminatorHead
    from agentgarten_b200.parallel.engine import ParallelConfig

    golden = probe("dmd", tmp_path / "dmd.pt")
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        from reference_probe import seeded_
    finally:
        sys.path.pop(0)
    config = tiny_config()
    plain = ParallelConfig(parameter_dtype="float32", fully_shard=False, activation_checkpointing="none",
                           compile=False)
    for kind in ("finite_difference", "exact"):
        want = golden[kind]
        towers = [build_network(config, init_device="cpu") for _ in range(3)]
        for index, tower in enumerate(towers):
            seeded_(tower, 20 + index)
        head = DiscriminatorHead(hidden_size=256, feature_layers=(0, 1), mlp_ratio=2.0, num_heads=4,
                                 init_device="cpu")
        for name, value in head.state_dict().items():  # the seeded head is the reference's head
            assert torch.equal(value, want["head"][name]), name
        model = DMDModel(
            student=towers[0], real_score=towers[1], fake_score=towers[2],
            conditioner=Cosmos3Conditioner(config=config, codec=None, geometry_noise_sigma=0.0,
                                           init_device="cpu", empty_prompt_ids=(3, 4, 5)),
            discriminator=head, gan=GANConfig(regularization=kind, warmup_updates=1),
            block_frames=4, fake_score_updates_per_student=2, student_parallel=plain,
            score_parallel=plain, discriminator_parallel=plain, seed=3)
        model.parallelize("cpu")
        seeded_(model.conditioner.text_encoder, 1)
        model.train()
        data = model.prepare_data_batch(batch_of(9, seed=8))
        for iteration in range(3):
            torch.manual_seed(100 + iteration)
            model.zero_grad(set_to_none=True)
            report, loss = model.training_step(data, iteration)
            loss.backward()
            expect = want[iteration]
            assert tuple(model.get_optimizer_names(iteration)) == tuple(expect["names"])
            assert float(loss) == pytest.approx(expect["loss"], rel=5e-5, abs=1e-7), (kind, iteration)
            for name, module in (("student", model.student), ("fake_score", model.fake_score),
                                 ("discriminator", head)):
                norm = sum(float(p.grad.double().square().sum()) for p in module.parameters()
                           if p.grad is not None) ** 0.5
                assert norm == pytest.approx(expect["grads"][name], rel=2e-4, abs=1e-9), (kind, iteration, name)
            mine = {k: float(v) for k, v in report.items() if torch.is_tensor(v) and v.numel() == 1}
            assert set(mine) == set(expect["report"]), (kind, iteration)
            for key, value in expect["report"].items():
                assert mine[key] == pytest.approx(value, rel=2e-4, abs=1e-6), (kind, iteration, key)
        model.eval()
        _, validation = model.validation_step(data, 0)
        assert float(validation) == pytest.approx(want["validation"], rel=5e-5)


def _ranks(script, *arguments, env, port, cwd):
    done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), *arguments],
                          capture_output=True, text=True, timeout=900, env=env, cwd=str(cwd))
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]


def test_checkpoints_interchange_with_the_reference(tmp_path):
    """Two Gloo ranks.  The reference (FSDP2, sharded optimizer state) trains two updates and
    saves ``iter_000000002``; this package resumes it and its third update gives the reference's
    third loss.  Then the reverse: this package saves, the reference resumes.  The two
    directories hold the same tensor keys."""
    from torch.distributed.checkpoint import FileSystemReader

    own_env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    own_env.update(AGB200_DISABLE_NATIVE="1", OMP_NUM_THREADS="2", PYTHONPATH=str(ROOT))
    probe_script = ROOT / "baseline" / "reference_probe.py"
    worker = ROOT / "tests" / "interchange_worker.py"
    theirs, mine = tmp_path / "reference_ckpt", tmp_path / "own_ckpt"

    _ranks(probe_script, "checkpoint", str(tmp_path / "a.pt"), "--directory", str(theirs),
           env=reference_env(), port=29671, cwd=ROOT / "baseline")
    _ranks(worker, str(tmp_path / "b.pt"), "--directory", str(theirs), "--resume",
           env=own_env, port=29672, cwd=ROOT)
    a, b = torch.load(tmp_path / "a.pt"), torch.load(tmp_path / "b.pt")
    assert b["loss"] == pytest.approx(a["loss"], rel=1e-6) and b["lr"] == pytest.approx(a["lr"])

    _ranks(worker, str(tmp_path / "c.pt"), "--directory", str(mine), env=own_env, port=29673, cwd=ROOT)
    _ranks(probe_script, "checkpoint", str(tmp_path / "d.pt"), "--directory", str(mine), "--resume",
           env=reference_env(), port=29674, cwd=ROOT / "baseline")
    c, d = torch.load(tmp_path / "c.pt"), torch.load(tmp_path / "d.pt")
    assert d["loss"] == pytest.approx(c["loss"], rel=1e-6) and d["lr"] == pytest.approx(c["lr"])
    assert c["loss"] == pytest.approx(a["loss"], rel=1e-6)  # the two runs are the same run

    keys = [set(FileSystemReader(str(d / "iter_000000002" / "tensor")).read_metadata().state_dict_metadata)
            for d in (theirs, mine)]
    assert keys[0] == keys[1], (sorted(keys[0] - keys[1])[:5], sorted(keys[1] - keys[0])[:5])
    assert (theirs / "latest").read_text() == (mine / "latest").read_text()
    assert sorted(p.name for p in (theirs / "iter_000000002").iterdir()) == \
        sorted(p.name for p in (mine / "iter_000000002").iterdir())


# Lines of a flattened recipe that may differ: options this package adds (AdaLN variant of the
# network, random weights for synthetic runs, the flat optimizer engine, the limit on skipped
# updates), classes that live in another module of this package, and default factories, which the
# reference's lazy call records as a placeholder and this package's as their value.
RECIPE_EXTENSIONS = re.compile(
    r"(geometry_mode|timestep_conditioning|special_tokens|codec\.architecture|random_init_seed|\.flat = None"
    r"|process_group = None|max_consecutive_skipped_updates|compile_options = <factory>|parallel\._target_"
    r"|gan\._target_)")


def test_pure_and_seeded_functions_equal_the_reference(tmp_path):
    """One probe file (``baseline/function_probe.py``) runs in the reference's process and in this
    one.  Equal bit for bit: rectified-flow utilities and the UniPC solver, learning-rate factors,
    geometry preprocessing with its seeded augmentations, media conversion and file names, history
    window, phase clock, stream positions, seeded discriminator and LoRA initialisation, the
    synthetic dataset and the stateful loader's order and cursor, a whole ``Trainer.train`` run on
    a toy model (parameter groups, clipping and spike events, metric names and values at every
    flush, validation, scheduler), and streams in all three position modes with eviction, a new
    prompt mid-stream and reference images; panels, defaults and refusals of ``sample()`` of the three objectives; raw
    batches through the conditioner (caption suffix, negative prompt, geometry pipeline, seeded
    latent noise, prompt dropout) with stand-ins for the VAE encoder and the tokenizer; periodic
    sampling inside a run (which batches, which options, untouched training streams) with the 120
    PNG files it leaves (names and bytes) and the writer's refusals and name rules; the codec
    wrapper's promises without weights; the objective base class (trainable patterns over aliased
    parameters, parameter groups, bindings and their refusals, a two-role step); weight overlays
    of ``train.model_initializations`` (released-weights directory, key patterns, several
    destinations, the resume subset, a run's checkpoint as source) and their plan; the optimizer
    on its CPU path (Adam / AdamW, without first or second moment, FP32 master weights under bf16
    parameters, per-group options, state round trip, refusals); the tables users and checkpoints
    depend on (key patterns of the released weights, LoRA module lists, configuration defaults,
    distillation endpoints, recipe constants) and the configuration trees of all seven recipes
    (every line, up to the options this package adds); tree mapping of tensors, seeding, mode and
    gradient-flag guards, atomic file helpers, image encoding, random-state capture; clipping
    helpers, lazy calls and their instantiation rules, rank helpers, the metric callback on odd step
    outputs and with a failing sink; resume under a changed recipe (the current recipe's rates,
    schedule and options win, progress comes back, no state is invented, components can be
    selected, the data cursor returns); the text tower on two prompts of different lengths; an
    update skipped for non-finite gradients (nothing steps, hook order, the next update goes
    through); what thirty constructors and entry points refuse, and in which words.  Equal
    to rounding: the restructured codecs (Wan 2.2 VAE, tiny decoders), a stream restarted on its
    kept arenas, the sampled latents and block-causal passes under bounded history windows and on
    a batch of two: these agree bit for bit in most runs, but the CPU kernels underneath do not
    promise the same rounding for the same values at another memory alignment (two runs of the
    reference alone can differ by 4e-7), so they are compared to 5e-5."""
    import importlib.util

    path = tmp_path / "functions.pt"
    done = subprocess.run([sys.executable, str(ROOT / "baseline" / "function_probe.py"), str(path)],
                          capture_output=True, text=True, timeout=1800, env=reference_env(),
                          cwd=str(ROOT / "baseline"))
    assert done.returncode == 0, done.stderr[-3000:]
    theirs = torch.load(path, weights_only=False)
    spec = importlib.util.spec_from_file_location("function_probe", ROOT / "baseline" / "function_probe.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    ours = module.collect()
    errors = {key: value for key, value in {**theirs, **ours}.items() if key.endswith("/error")}
    assert not errors, errors
    assert sorted(ours) == sorted(theirs)
    assert len(ours) > 600

    def to_rounding(key: str) -> bool:
        return key.startswith(("vae/", "tiny/", "window/", "batched/forward")) or key.endswith("/restart") \
            or (key.startswith("sampling/") and key.endswith("/sample"))

    for key, want in theirs.items():
        got = ours[key]
        if key == "constants/config":   # this package's network has two more options (AdaLN variant)
            assert set(want) <= set(got), (key, sorted(set(want) - set(got)))
            continue
        if key.startswith("recipes/"):
            assert isinstance(want, list) and isinstance(got, list), (key, want if isinstance(want, str) else got)
            stray = sorted(line for line in set(want) ^ set(got) if not RECIPE_EXTENSIONS.search(line))
            assert not stray and len(got) > 250, (key, stray[:10])
            continue
        if not torch.is_tensor(want):
            assert got == want, (key, got, want)
            continue
        assert torch.is_tensor(got) and got.shape == want.shape and got.dtype == want.dtype, key
        if to_rounding(key):
            assert torch.allclose(got, want, atol=5e-5, rtol=1e-5), (key, float((got - want).abs().max()))
        else:
            assert torch.equal(torch.nan_to_num(got), torch.nan_to_num(want)), \
                (key, float((torch.nan_to_num(got.double()) - torch.nan_to_num(want.double())).abs().max()))
            if want.is_floating_point():
                assert torch.equal(torch.isnan(got), torch.isnan(want)), key


def test_exported_artifacts_interchange_with_the_reference(tmp_path):
    """``save_artifact`` of either tree is read by ``inspect_artifact`` / ``load_artifact`` of the
    other: same files, same manifest, every tensor of the student (with declared LoRA) and of the
    text tower equal, iteration, caption horizon and LoRA declaration carried over."""
    import importlib.util
    import json

    spec = importlib.util.spec_from_file_location("function_probe", ROOT / "baseline" / "function_probe.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    ours_dir, theirs_dir = tmp_path / "ours", tmp_path / "theirs"
    saved = module.artifact_exchange(str(ours_dir))
    path = tmp_path / "exchange.pt"
    done = subprocess.run([sys.executable, str(ROOT / "baseline" / "function_probe.py"), str(path), "artifact",
                           str(theirs_dir), str(ours_dir)], capture_output=True, text=True, timeout=900,
                          env=reference_env(), cwd=str(ROOT / "baseline"))
    assert done.returncode == 0, done.stderr[-3000:]
    theirs = torch.load(path, weights_only=False)           # the reference read this package's export
    ours = module.artifact_exchange(str(tmp_path / "again"), str(theirs_dir))   # and the reverse
    assert saved["saved/files"] == theirs["saved/files"] == ["config.yaml", "manifest.json",
                                                             "student.safetensors", "und.safetensors"]
    assert json.loads((ours_dir / "manifest.json").read_text()) == json.loads((theirs_dir / "manifest.json").read_text())
    for key in ("saved/student_keys", "saved/text_keys", "loaded/iteration", "loaded/frames", "loaded/lora",
                "loaded/tokenizer", "loaded/report"):
        assert ours[key] == theirs[key], key
    assert ours["loaded/iteration"] == 42 and ours["loaded/frames"] == 13
    assert set(theirs["loaded/config"]) <= set(ours["loaded/config"])   # this package has two more options
    tensors = [key for key in theirs if key.startswith(("loaded/student/", "loaded/text/"))]
    assert len(tensors) > 40 and sorted(tensors) == sorted(k for k in ours if k.startswith(("loaded/student/",
                                                                                             "loaded/text/")))
    for key in tensors:
        assert torch.equal(ours[key], theirs[key]), key


def test_data_parallel_wrapper_equals_the_reference(tmp_path):
    """Two Gloo ranks in each tree: loss closures through ``wrap_ddp`` with two micro-batches per
    update.  Losses, the local gradients after the first micro-batch, the averaged ones after the
    last, and the parameters after every step are equal bit for bit between the trees; inside a
    tree the ranks end every update with the same parameters."""
    results = []
    for label, env, port in (("theirs", reference_env(), 29721),
                             ("ours", dict(os.environ, PYTHONPATH=str(ROOT), AGB200_DISABLE_NATIVE="1"), 29722)):
        env = {k: v for k, v in env.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
        env["OMP_NUM_THREADS"] = "2"
        path = tmp_path / f"{label}.pt"
        done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                               "--master-addr", "127.0.0.1", "--master-port", str(port),
                               str(ROOT / "baseline" / "function_probe.py"), str(path), "ddp"],
                              capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT / "baseline"))
        assert done.returncode == 0 and path.exists(), done.stderr[-3000:]
        results.append(torch.load(path, weights_only=False))
    theirs, ours = results
    assert sorted(theirs) == sorted(ours) and len(ours) == 16
    for key, want in theirs.items():
        got = ours[key]
        assert torch.equal(got, want) if torch.is_tensor(want) else got == want, key
    assert ours["ddp/0/updated"] == [False, False] and ours["ddp/1/updated"] == [True, True]
    assert not torch.equal(ours["ddp/0/gradients"][0], ours["ddp/0/gradients"][1])     # still local
    for micro in (1, 3):
        assert torch.equal(ours[f"ddp/{micro}/weights"][0], ours[f"ddp/{micro}/weights"][1])


def test_batch_transport_equals_the_reference(tmp_path):
    """Four Gloo ranks in context-parallel groups of two, in each tree: which member reads which
    micro-batch, the tensors, nested structure and random state the other member receives, the
    common end of the data, and a dataset failure on one rank that every rank reports."""
    results = []
    for label, env, port in (("theirs", reference_env(), 29723),
                             ("ours", dict(os.environ, PYTHONPATH=str(ROOT), AGB200_DISABLE_NATIVE="1"), 29724)):
        env = {k: v for k, v in env.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
        env["OMP_NUM_THREADS"] = "2"
        path = tmp_path / f"{label}.pt"
        done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                               "--master-addr", "127.0.0.1", "--master-port", str(port),
                               str(ROOT / "baseline" / "function_probe.py"), str(path), "transport"],
                              capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT / "baseline"))
        assert done.returncode == 0 and path.exists(), done.stderr[-3000:]
        results.append(torch.load(path, weights_only=False))
    theirs, ours = results
    assert sorted(theirs) == sorted(ours) and len(ours) == 44
    for key, want in theirs.items():
        got = ours[key]
        assert torch.equal(got, want) if torch.is_tensor(want) else got == want, key
    assert all(ours[f"transport/{member}/failure"] == "(True, True)" for member in range(4))
    # both members of a group hold the same prepared batch and continue with the same streams
    for pair in ((0, 1), (2, 3)):
        for step in range(3):
            for part in ("meta", "tensors"):
                a, b = (ours[f"transport/{member}/{step}/{part}"] for member in pair)
                assert torch.equal(a, b) if torch.is_tensor(a) else a == b, (pair, step, part)


def test_training_runs_are_served_by_either_tree(tmp_path):
    """A run directory (checkpoint, resolved configuration, the released text tower it names) laid
    out by one tree is inspected and loaded for serving by the other: the same overlay order,
    caption horizon, tokenizer location, progress reports and every tensor of both towers."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("function_probe", ROOT / "baseline" / "function_probe.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    ours_run, theirs_run = tmp_path / "ours", tmp_path / "theirs"
    laid_out = module.run_exchange(str(ours_run))
    path = tmp_path / "exchange.pt"
    done = subprocess.run([sys.executable, str(ROOT / "baseline" / "function_probe.py"), str(path), "run",
                           str(theirs_run), str(ours_run)], capture_output=True, text=True, timeout=900,
                          env=reference_env(), cwd=str(ROOT / "baseline"))
    assert done.returncode == 0, done.stderr[-3000:]
    theirs = torch.load(path, weights_only=False)            # the reference served this package's run
    ours = module.run_exchange(str(tmp_path / "again"), str(theirs_run))    # and the reverse
    assert laid_out["run/files"] == theirs["run/files"] == ours["run/files"]
    assert sorted(ours) == sorted(theirs) and len(ours) == 60
    assert ours["run/spec"][:2] == [5, 9] and ours["run/frozen"] is True
    for key, want in theirs.items():
        got = ours[key]
        assert torch.equal(got, want) if torch.is_tensor(want) else got == want, key
