"""Weights & Biases sinks for metrics and sample videos.

Runs are shared per process through a registry keyed by (project, name, directory); every
sink holds a reference and the run is finished when the last one closes.  The metric sink
can hand its writes to a queue drained by a background thread, so a slow network never
stalls a training step.  The ``wandb`` package is imported lazily; without it (or when
``mode="disabled"``) the sinks do nothing.

Parity: reference ``wm/infra/callbacks/wandb.py:31-354``.
"""

from __future__ import annotations

import queue
import threading
from collections.abc import Mapping
from typing import Any

from agentgarten_b200.infra.distributed import is_rank0
from agentgarten_b200.utils import log

from .media import ImageVideoArtifactWriter

__all__ = ["WandbArtifactWriter", "WandbMetricSink"]

_lock = threading.Lock()
_runs: dict[tuple, list] = {}   # key -> [run, reference count]


def _acquire(project: str | None, name: str | None, directory: str | None, mode: str,
             config: Mapping[str, Any] | None, extra: Mapping[str, Any]):
    if mode == "disabled" or not is_rank0():
        return None, None
    try:
        import wandb
    except ImportError:
        log.warning("wandb is not installed; W&B sinks are disabled.")
        return None, None
    key = (project, name, directory)
    with _lock:
        entry = _runs.get(key)
        if entry is None:
            run = wandb.init(project=project, name=name, dir=directory, mode=mode,
                             config=dict(config or {}), reinit=True, **dict(extra))
            entry = _runs[key] = [run, 0]
        entry[1] += 1
        return key, entry[0]


def _release(key) -> None:
    if key is None:
        return
    with _lock:
        entry = _runs.get(key)
        if entry is None:
            return
        entry[1] -= 1
        if entry[1] <= 0:
            _runs.pop(key, None)
            try:
                entry[0].finish()
            except Exception as error:
                log.warning(f"wandb run finish failed: {type(error).__name__}: {error}")


class WandbMetricSink:
    def __init__(self, *, project: str | None = None, name: str | None = None, dir: str | None = None,
                 mode: str = "online", config: Mapping[str, Any] | None = None,
                 async_write: bool = True, queue_size: int = 256, **init_kwargs: Any) -> None:
        self._key, self._run = _acquire(project, name, dir, mode, config, init_kwargs)
        self._queue: queue.Queue | None = None
        self._thread: threading.Thread | None = None
        if self._run is not None and async_write:
            self._queue = queue.Queue(maxsize=int(queue_size))
            self._thread = threading.Thread(target=self._drain, name="wandb-metrics", daemon=True)
            self._thread.start()

    def _drain(self) -> None:
        while True:
            item = self._queue.get()
            if item is None:
                return
            metrics, iteration = item
            try:
                self._run.log(metrics, step=iteration)
            except Exception as error:
                log.warning(f"wandb log failed: {type(error).__name__}: {error}")

    def write(self, metrics: Mapping[str, float], *, iteration: int) -> None:
        if self._run is None:
            return
        if self._queue is not None:
            self._queue.put((dict(metrics), int(iteration)))
        else:
            self._run.log(dict(metrics), step=int(iteration))

    def close(self) -> None:
        if self._queue is not None:
            self._queue.put(None)
            self._thread.join(timeout=60)
            self._queue = None
        _release(self._key)
        self._key = self._run = None


class WandbArtifactWriter:
    """Logs the comparison video of a sample (encoded once by the media writer's code)."""

    def __init__(self, *, project: str | None = None, name: str | None = None, dir: str | None = None,
                 mode: str = "online", key: str = "samples/comparison", fps: int = 16,
                 media: ImageVideoArtifactWriter | None = None, **init_kwargs: Any) -> None:
        self._key, self._run = _acquire(project, name, dir, mode, None, init_kwargs)
        self.key, self.fps = key, int(fps)
        self.media = media or ImageVideoArtifactWriter(fps=fps, save_individual_artifacts=False)

    def write(self, value: Any, *, output_dir: str, split: str, iteration: int, rank: int,
              sample_batch_index: int = 0) -> None:
        if self._run is None:
            return
        import wandb

        from agentgarten_b200.utils import io

        for name, b, _batch, pixels in self.media._artifacts(value):
            if pixels.shape[0] == 1:
                item = wandb.Image(pixels[0].numpy())
            else:
                clip = io.encode_video(pixels.numpy(), fps=self.fps, quality=5)
                item = wandb.Video(clip, format="mp4")
            self._run.log({f"{self.key}/{split}/{name}_{sample_batch_index:02d}_{b:02d}": item},
                          step=int(iteration))

    def close(self) -> None:
        _release(self._key)
        self._key = self._run = None
