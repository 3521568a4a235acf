"""Sections every experiment starts from.

``job`` (output dir), ``runtime`` (device, backend, process-group timeout, seeding, torch
backend flags), ``model`` / ``optimizer`` / ``scheduler`` (mandatory, ``???``), ``trainer``
(accumulation 1; callbacks ``grad_monitor`` then ``metrics`` — the monitor publishes
gradient norms into the step outputs before the metric callback reads them),
``checkpoint`` (async thread mode), a disabled ``grad_scaler``, loaders and ``train``.

Parity: reference ``wm/configs/base.py:16-80``.
"""

from __future__ import annotations

import torch

from agentgarten_b200.infra.callbacks import GradClipMonitor, LoguruMetricSink, ScalarMetricCallback
from agentgarten_b200.infra.checkpoint import DistributedCheckpointer
from agentgarten_b200.infra.config import ConfigNode, LazyCall, LazyDict
from agentgarten_b200.infra.trainer import Trainer

__all__ = ["make_base_config"]


def make_base_config() -> LazyDict:
    return ConfigNode({
        "job": {"output_dir": "???"},
        "runtime": {
            "device": "cuda",
            "backend": "nccl",
            "process_group_timeout_seconds": 300.0,
            "seed": 0,
            "seed_by_rank": True,
            "torch": {"benchmark": True, "allow_tf32": True, "float32_matmul_precision": "high",
                      "compile": {"recompile_limit": 32, "use_duck_shape": False}},
        },
        "model": "???",
        "optimizer": "???",
        "scheduler": "???",
        "trainer": LazyCall(Trainer)(
            grad_accum_steps=1,
            callbacks={
                "grad_monitor": LazyCall(GradClipMonitor)(
                    max_norm=1.0, spike_threshold=10.0, spike_ratio=5.0, warmup_updates=10,
                    output_dir="${job.output_dir}/diagnostics/grad_spikes"),
                "metrics": LazyCall(ScalarMetricCallback)(
                    every_n=10, report_update_speed=True, sinks=[LazyCall(LoguruMetricSink)()]),
            }),
        "checkpoint": LazyCall(DistributedCheckpointer)(
            save_dir="${job.output_dir}/checkpoints", async_mode="thread",
            async_timeout_seconds=3600.0),
        "grad_scaler": LazyCall(torch.amp.GradScaler)(device="cuda", enabled=False),
        "dataloader_train": "???",
        "dataloader_val": None,
        "model_wrapper": None,
        "train": {
            "max_iterations": 10_000,
            "model_initializations": {},
            "checkpoint_path": None,
            "checkpoint_components": None,
            "checkpoint_optimizer_names": None,
            "checkpoint_scheduler_names": None,
            "checkpoint_interval": 500,
            "validation_interval": 500,
            "max_val_steps": 8,
            "validate_at_start": True,
            "save_final_checkpoint": True,
            "runtime_metadata": None,
        },
    })
