"""Recipe composition and the whole training entry point on CPU (one rank and two gloo ranks)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from agentgarten_b200.configs.compose import compose_config
from agentgarten_b200.infra.config import ConfigError, instantiate

ROOT = Path(__file__).resolve().parents[1]
RECIPES = ["bidirectional", "ar_teacher_forcing", "ar_diffusion_forcing", "dmd", "dmd_gan",
           "dmd_gan_exact", "dmd_gan_lora"]


@pytest.mark.parametrize("name", RECIPES)
def test_released_recipes_compose(name):
    config = compose_config([f"experiment=cosmos3/{name}", "trainer.grad_accum_steps=3",
                             "model_parallel.context_parallel_size=2"])
    assert config.experiment == f"cosmos3/{name}"
    assert config.trainer.grad_accum_steps == 3
    parallel_nodes = [v for k, v in config.model.items() if k.endswith("parallel") and v is not None]
    assert parallel_nodes and all(node.context_parallel_size == 2 for node in parallel_nodes)
    assert config.job.output_dir.endswith(name) and "${" not in config.job.output_dir
    assert config.cosmos3.hidden_size == 4096 and config.cosmos3.num_hidden_layers == 36
    assert "grad_monitor" in config.trainer.callbacks and "samples" in config.trainer.callbacks
    assert config.model._target_.startswith("agentgarten_b200.models.")


def test_selector_rules():
    with pytest.raises(ValueError):
        compose_config(["trainer.grad_accum_steps=2"])
    with pytest.raises(ValueError):
        compose_config(["experiment=cosmos3/bidirectional", "experiment=cosmos3/dmd"])
    with pytest.raises(ValueError):
        compose_config(["experiment=bidirectional"])
    with pytest.raises(ModuleNotFoundError):
        compose_config(["experiment=cosmos3/does_not_exist"])
    with pytest.raises(ConfigError):
        compose_config(["experiment=synthetic/tiny"])  # job.output_dir is mandatory


def test_wm_alias_runs_the_same_recipes():
    import wm.configs.compose as alias
    config = alias.compose_config(["experiment=cosmos3/bidirectional"],
                                  experiment_module_root="wm.configs.experiments")
    assert config.trainer.grad_accum_steps == 4


def _train(args, tmp_path, ranks=1, port=29631):
    env = dict(os.environ, PYTHONPATH=str(ROOT), AGB200_DISABLE_NATIVE="1")
    base = [sys.executable]
    if ranks > 1:
        base += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
                 "--master-addr", "127.0.0.1", "--master-port", str(port)]
    cmd = base + ["-m", "agentgarten_b200.train", "experiment=synthetic/tiny",
                  f"job.output_dir={tmp_path}", "runtime.device=cpu", "runtime.backend=gloo", *args]
    Path(tmp_path).mkdir(parents=True, exist_ok=True)
    done = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    return done.stdout + done.stderr


def _losses(text):
    out = {}
    for line in text.splitlines():
        if "train/loss=" in line and "iteration=" in line:
            step = int(line.split("iteration=")[1].split()[0])
            out[step] = float(line.split("train/loss=")[1].split()[0])
    return out


def test_train_checkpoint_resume_continues_the_same_run(tmp_path):
    straight = _losses(_train(["train.max_iterations=6"], tmp_path / "a"))
    assert sorted(straight) == [1, 2, 3, 4, 5, 6]
    saved = tmp_path / "a" / "checkpoints"
    assert (saved / "latest").read_text().strip().endswith("6")
    assert (tmp_path / "a" / "config.yaml").is_file()
    # stop after three updates, then resume to six: same losses as the uninterrupted run
    _train(["train.max_iterations=3"], tmp_path / "b")
    resumed = _losses(_train(["train.max_iterations=6", "train.checkpoint_path=latest"], tmp_path / "b"))
    assert sorted(resumed) == [4, 5, 6]
    for step in (4, 5, 6):
        assert resumed[step] == pytest.approx(straight[step], rel=1e-5), (step, resumed, straight)


def test_two_ranks_train_and_shard_the_optimizer(tmp_path):
    text = _train(["train.max_iterations=3", "train.checkpoint_interval=3"], tmp_path, ranks=2)
    losses = _losses(text)
    assert sorted(losses) == [1, 2, 3] and all(torch.isfinite(torch.tensor(v)) for v in losses.values())
    assert (tmp_path / "checkpoints" / "iter_000000003" / "dataloader" / "rank_00001.pt").is_file()


def test_persistent_nonfinite_gradients_stop_the_run():
    from agentgarten_b200.infra.trainer import Trainer
    assert Trainer(max_consecutive_skipped_updates=5).max_consecutive_skipped_updates == 5
