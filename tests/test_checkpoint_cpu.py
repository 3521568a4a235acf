import torch

from agentgarten_b200.data.loader import StatefulDataLoader
from agentgarten_b200.data.video import SyntheticLatentDataset
from agentgarten_b200.infra.checkpoint import DistributedCheckpointer
from agentgarten_b200.infra.checkpoint.plan import build_model_restore_plan, plan_model_initializations
from agentgarten_b200.infra.optim import FusedAdam, LinearWarmup
from agentgarten_b200.models.diffusion import DiffusionModel

from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network


def _job(seed=0):
    cfg = tiny_config()
    model = DiffusionModel(net=tiny_network(cfg, seed=seed), conditioner=tiny_conditioner(cfg),
                           text_dropout=0.0)
    model.parallelize("cpu")
    opt = FusedAdam(model._group_trainable_parameters(), lr=1e-3, use_te_capturable_kernel=True,
                    master_weights=True)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, LinearWarmup(warmup_steps=10, start_factor=0.1))
    model.optimizer_dict, model.scheduler_dict = {"net": opt}, {"net": sched}
    return model, opt, sched


def _step(model, opt, sched, batch, seed):
    g = torch.Generator().manual_seed(seed)
    _, loss = model._objective(batch, g, None)
    loss.backward()
    opt.step()
    sched.step()
    opt.zero_grad()
    return float(loss)


def test_save_resume_continues_exactly(tmp_path):
    model, opt, sched = _job()
    batch = model.prepare_data_batch(synthetic_batch())
    loader = StatefulDataLoader(SyntheticLatentDataset(length=8, latent_frames=5, latent_height=8,
                                                       latent_width=8, text_tokens=6, vocab_size=100),
                                batch_size=2, shuffle=True, seed=3)
    it = iter(loader)
    next(it)
    for s in range(3):
        _step(model, opt, sched, batch, s)
    saver = DistributedCheckpointer(tmp_path / "ckpt", async_mode="thread")
    torch.manual_seed(123)
    saver.save(model, {"net": opt}, {"net": sched}, None, iteration=3, dataloader=loader)
    saver.finalize()
    assert (tmp_path / "ckpt" / "latest").read_text().strip() == "iter_000000003"
    assert (tmp_path / "ckpt" / "iter_000000003" / "tensor" / ".metadata").is_file()
    assert (tmp_path / "ckpt" / "iter_000000003" / "metadata.json").is_file()
    expected_rand = torch.rand(3)
    reference = [_step(model, opt, sched, batch, 10 + s) for s in range(2)]

    fresh, opt2, sched2 = _job(seed=5)
    loader2 = StatefulDataLoader(loader.dataset, batch_size=2, shuffle=True, seed=3)
    loader_ckpt = DistributedCheckpointer(tmp_path / "ckpt", async_mode=None)
    result = loader_ckpt.load(fresh, {"net": opt2}, {"net": sched2}, None, path="latest", dataloader=loader2)
    assert result.iteration == 3 and "model" in result.loaded_components
    assert not result.missing_model_keys and not result.unexpected_model_keys
    assert loader2.state_dict() == {"epoch": 0, "batch_offset": 1}
    assert sched2.last_epoch == 3 and abs(opt2.param_groups[0]["lr"] - 1e-3 * (0.1 + 0.9 * 0.3)) < 1e-12
    assert loader_ckpt.restore_pending_rng_state()
    assert torch.equal(torch.rand(3), expected_rand)
    resumed = [_step(fresh, opt2, sched2, batch, 10 + s) for s in range(2)]
    assert resumed == reference
    # the frozen conditioner is not part of a checkpoint
    keys = torch.distributed.checkpoint.FileSystemReader(
        str(tmp_path / "ckpt" / "iter_000000003" / "tensor")).read_metadata().state_dict_metadata
    assert not any(k.startswith("model.conditioner.") for k in keys)
    assert any(k.startswith("optimizers.net.state.net.layers.0.") and k.endswith("master_param") for k in keys)


def test_overlay_into_several_prefixes(tmp_path):
    import torch.distributed.checkpoint as dcp

    cfg = tiny_config()
    donor = tiny_network(cfg, seed=9)
    dcp.save({k: v for k, v in donor.state_dict().items()},
             storage_writer=dcp.FileSystemWriter(str(tmp_path / "donor")))
    model, *_ = _job(seed=1)
    before = model.net.layers[1].mlp_moe_gen.up_proj.weight.clone()
    inits = {"net": {"path": str(tmp_path / "donor"), "model_key_prefixes": ["net"],
                     "source_model_key_prefix": "",
                     "source_model_key_patterns": [r"layers\.0\..*", r"proj_(?:in|out)\.(?:weight|bias)"],
                     "resume_model_key_prefixes": None}}
    DistributedCheckpointer(tmp_path / "x", async_mode=None).initialize_model(model, inits)
    bf16 = torch.bfloat16
    assert torch.equal(model.net.layers[0].mlp_moe_gen.up_proj.weight, donor.layers[0].mlp_moe_gen.up_proj.weight.to(bf16))
    assert torch.equal(model.net.proj_in.weight, donor.proj_in.weight.to(bf16))
    assert torch.equal(model.net.layers[1].mlp_moe_gen.up_proj.weight, before)
    assert plan_model_initializations(inits, resume=True) == ()


def test_restore_plan_rules():
    plan = build_model_restore_plan(live_keys=["a.w", "b.w", "c"], saved_keys=["w", "z"], overlay=True,
                                    source_prefix="", destination_prefixes=["a", "b"],
                                    source_patterns=[r"w"])
    assert plan.entries[0].targets == ("a.w", "b.w") and plan.missing_model_keys == ()
    strict = build_model_restore_plan(live_keys=["x", "y"], saved_keys=["y", "q"], overlay=False)
    assert strict.missing_model_keys == ("x",) and strict.unexpected_model_keys == ("q",)
    merged = plan_model_initializations(
        {"s": {"path": "p", "model_key_prefixes": ["student"], "source_model_key_prefix": ""},
         "f": {"path": "p", "model_key_prefixes": ["fake"], "source_model_key_prefix": ""}}, resume=False)
    assert len(merged) == 1 and merged[0].destinations == ("student", "fake")


# ------------------------------------------------------------------ failures on the host
def test_failed_write_never_publishes_latest(tmp_path, monkeypatch):
    """The tensor write fails (a full disk, a dead mount): the error surfaces at finalize and
    the `latest` pointer keeps naming the last good checkpoint."""
    import pytest
    import torch.distributed.checkpoint as dcp

    model, opt, sched = _job()
    saver = DistributedCheckpointer(tmp_path / "ckpt", async_mode=None)
    saver.save(model, {"net": opt}, {"net": sched}, None, iteration=1)
    assert (tmp_path / "ckpt" / "latest").read_text().strip() == "iter_000000001"

    def broken(*args, **kwargs):
        raise OSError("No space left on device")

    monkeypatch.setattr(dcp, "save", broken)
    with pytest.raises(RuntimeError, match="No space left"):
        saver.save(model, {"net": opt}, {"net": sched}, None, iteration=2)
    assert (tmp_path / "ckpt" / "latest").read_text().strip() == "iter_000000001"
    # error shutdown: nothing collective, nothing raised, nothing published
    saver.finalize_after_error()
    assert (tmp_path / "ckpt" / "latest").read_text().strip() == "iter_000000001"


def test_async_save_that_stalls_or_fails_is_reported_at_the_next_finalize(tmp_path, monkeypatch):
    """The background write never finishes (a hung mount) or fails in its thread: the save call
    itself returns, the error surfaces at ``finalize`` (a time-out after ``async_timeout_seconds``
    in the first case) and `latest` still names the last complete checkpoint."""
    from concurrent.futures import Future

    import pytest
    import torch.distributed.checkpoint as dcp

    model, opt, sched = _job()
    saver = DistributedCheckpointer(tmp_path / "ckpt", async_mode="thread")
    saver.save(model, {"net": opt}, {"net": sched}, None, iteration=1)
    saver.finalize()
    saver.async_timeout_seconds = 0.2                  # from here on a write gets 0.2 s
    pointer = tmp_path / "ckpt" / "latest"
    assert pointer.read_text().strip() == "iter_000000001"

    never = Future()                                   # a write that does not come back
    monkeypatch.setattr(dcp, "async_save", lambda *args, **kwargs: never)
    saver.save(model, {"net": opt}, {"net": sched}, None, iteration=2)       # returns at once
    with pytest.raises(RuntimeError, match="iter_000000002"):
        saver.finalize()
    assert pointer.read_text().strip() == "iter_000000001"

    failed = Future()
    failed.set_exception(OSError("Input/output error"))
    monkeypatch.setattr(dcp, "async_save", lambda *args, **kwargs: failed)
    saver.save(model, {"net": opt}, {"net": sched}, None, iteration=3)
    with pytest.raises(RuntimeError, match="Input/output error"):
        saver.save(model, {"net": opt}, {"net": sched}, None, iteration=4)   # waits for 3 first
    assert pointer.read_text().strip() == "iter_000000001"
    saver.finalize_after_error()                       # nothing pending any more, nothing raised


def test_failed_latest_publication_is_reported(tmp_path, monkeypatch):
    import pytest

    from agentgarten_b200.infra.checkpoint import checkpointer as module

    model, opt, sched = _job()
    saver = DistributedCheckpointer(tmp_path / "ckpt", async_mode=None)

    def broken(text, path):
        raise PermissionError("read-only file system")

    monkeypatch.setattr(module, "atomic_put_text", broken)
    with pytest.raises(RuntimeError, match="latest pointer publication"):
        saver.save(model, {"net": opt}, {"net": sched}, None, iteration=4)
    assert not (tmp_path / "ckpt" / "latest").exists()


def test_truncated_shard_fails_the_load_loudly(tmp_path):
    import pytest

    model, opt, sched = _job()
    saver = DistributedCheckpointer(tmp_path / "ckpt", async_mode=None)
    saver.save(model, {"net": opt}, {"net": sched}, None, iteration=1)
    shard = next((tmp_path / "ckpt" / "iter_000000001" / "tensor").glob("*.distcp"))
    data = shard.read_bytes()
    shard.write_bytes(data[: len(data) // 3])
    fresh, opt2, sched2 = _job(seed=7)
    with pytest.raises(Exception):
        DistributedCheckpointer(tmp_path / "ckpt", async_mode=None).load(fresh, {"net": opt2}, {"net": sched2}, None,
                                                                        path="latest")


def test_load_path_semantics(tmp_path):
    """``None`` loads nothing (even when ``latest`` exists), the literal ``"latest"`` follows the
    pointer and fails without one, an absolute pointer target is honoured, and a directory
    path names the checkpoint itself."""
    import pytest

    model, opt, sched = _job()
    saver = DistributedCheckpointer(tmp_path / "ckpt", async_mode=None)
    with pytest.raises(FileNotFoundError, match="No latest checkpoint pointer"):
        saver.load(model, {"net": opt}, {"net": sched}, None, path="latest")
    saver.save(model, {"net": opt}, {"net": sched}, None, iteration=2)
    saver.finalize()
    fresh, opt2, sched2 = _job(seed=7)
    result = saver.load(fresh, {"net": opt2}, {"net": sched2}, None, path=None)
    assert result.iteration == 0 and result.loaded_components == ()
    result = saver.load(fresh, {"net": opt2}, {"net": sched2}, None, path="latest")
    assert result.iteration == 2 and "model" in result.loaded_components
    fresh, opt2, sched2 = _job(seed=8)
    result = saver.load(fresh, {"net": opt2}, {"net": sched2}, None, path=tmp_path / "ckpt" / "iter_000000002")
    assert result.iteration == 2
    # an absolute pointer target, from a checkpointer whose save_dir is elsewhere
    other = DistributedCheckpointer(tmp_path / "elsewhere", async_mode=None)
    (tmp_path / "elsewhere").mkdir()
    (tmp_path / "elsewhere" / "latest").write_text(str(tmp_path / "ckpt" / "iter_000000002") + "\n")
    fresh, opt2, sched2 = _job(seed=9)
    assert other.load(fresh, {"net": opt2}, {"net": sched2}, None, path="latest").iteration == 2
    (tmp_path / "elsewhere" / "latest").write_text("\n")
    with pytest.raises(FileNotFoundError, match="empty"):
        other.load(fresh, {"net": opt2}, {"net": sched2}, None, path="latest")
