"""Weights & Biases sinks for scalar metrics and sample media.

All sinks of a process write into ONE run: the SDK keeps a single global run, so the first sink
that needs it starts it (after ``wandb.login`` when ``WANDB_API_KEY`` is set) or adopts a run the
process already has, the others attach, and the sink that closes last finishes a run this module
started.  Nothing touches the SDK before the first write: building a config, a dry run or a
non-zero rank never imports ``wandb``.  Every SDK call happens under one lock, because the metric
sink may drain its queue on a worker thread while a validation pass logs media.

``WandbMetricSink(async_write=True)`` hands its payloads to that worker so that a slow service
never stalls an update; after a failed write the worker drops what is queued and the sink stays
quiet (training goes on).  ``step_metrics`` maps metric patterns to the metric that is their
x-axis (``wandb.define_metric``).

Parity: reference ``wm/infra/callbacks/wandb.py:31-354`` (constructor arguments, lazy start,
shared run, key layout ``<split>/batch_<index>/<artifact>[/<sample>]``, pre-encoded mp4).
"""

from __future__ import annotations

import importlib
import os
import threading
from collections.abc import Mapping, Sequence
from queue import SimpleQueue
from typing import Any

from agentgarten_b200.infra.distributed import is_rank0
from agentgarten_b200.utils import io, log

from .media import ImageVideoArtifactWriter

__all__ = ["WandbArtifactWriter", "WandbMetricSink"]

_sdk_lock = threading.RLock()   # guards the attachment table and every SDK call


class _ProcessRun:
    """The one run of this process and the sinks attached to it."""

    sdk: Any = None
    run: Any = None
    started_here = False
    attached: set[int] = set()

    @classmethod
    def attach(cls, client: "_RunClient") -> Any:
        """The SDK module with a live run for ``client`` (started or adopted on first use)."""
        if cls.sdk is None:
            try:
                cls.sdk = importlib.import_module("wandb")
            except ModuleNotFoundError as error:
                if error.name != "wandb":
                    raise
                raise ModuleNotFoundError(
                    "W&B logging requires the optional dependency; install wm[wandb]") from error
        sdk = cls.sdk
        cls.attached.add(id(client))
        if cls.run is None:
            if getattr(sdk, "run", None) is not None:
                cls.run, cls.started_here = sdk.run, False       # the process already has a run
            else:
                key = os.environ.get("WANDB_API_KEY")
                if key:
                    sdk.login(key=key, relogin=False)
                try:
                    sdk.init(project=client.project, group=client.group, name=client.name,
                             mode=client.mode)
                finally:   # a half-started run is ours to finish as well
                    cls.run = getattr(sdk, "run", None)
                    cls.started_here = cls.run is not None
        if getattr(sdk, "run", None) is not cls.run:
            raise RuntimeError("The shared W&B run was replaced or finished externally")
        return sdk

    @classmethod
    def detach(cls, client: "_RunClient") -> None:
        cls.attached.discard(id(client))
        if cls.attached or cls.sdk is None:
            return
        sdk, run, ours = cls.sdk, cls.run, cls.started_here
        cls.sdk, cls.run, cls.started_here = None, None, False
        if ours and run is not None and getattr(sdk, "run", None) is run:
            sdk.finish()


class _RunClient:
    def __init__(self, project: str, group: str | None = None, name: str | None = None,
                 mode: str | None = None, step_metrics: Mapping[str, str] | None = None) -> None:
        self.project, self.group, self.name, self.mode = project, group, name, mode
        self.step_metrics = dict(step_metrics or {})
        self._closed = False
        self._axes_defined = False

    def _initialize(self) -> Any | None:
        """The SDK, with the run started and this sink's x-axes declared; None once closed."""
        with _sdk_lock:
            if self._closed:
                return None
            sdk = _ProcessRun.attach(self)
            if not self._axes_defined:
                define = getattr(sdk, "define_metric", None)
                if callable(define):
                    for pattern, axis in self.step_metrics.items():
                        define(pattern, step_metric=axis)
                self._axes_defined = True
            return sdk

    def _log(self, payload: Mapping[str, Any], *, iteration: int) -> None:
        with _sdk_lock:
            sdk = self._initialize()
            if sdk is not None:
                sdk.log(dict(payload), step=int(iteration))

    def close(self) -> None:
        if not is_rank0():
            return
        with _sdk_lock:
            if self._closed:
                return
            self._closed = True
            _ProcessRun.detach(self)


class WandbMetricSink(_RunClient):
    def __init__(self, project: str, group: str | None = None, name: str | None = None,
                 mode: str | None = None, *, async_write: bool = False,
                 step_metrics: Mapping[str, str] | None = None) -> None:
        super().__init__(project=project, group=group, name=name, mode=mode, step_metrics=step_metrics)
        self.async_write = bool(async_write)
        self._inbox: SimpleQueue | None = None
        self._worker: threading.Thread | None = None
        self._worker_error: BaseException | None = None
        self._gate = threading.Lock()      # write() against close()
        self._closing = False

    _STOP = object()

    def _give_up(self, error: BaseException) -> None:
        self._worker_error = error
        log.warning("Disabling asynchronous W&B metric writes after failure: "
                    f"{type(error).__name__}: {error}")

    def _drain(self) -> None:
        inbox = self._inbox
        for item in iter(inbox.get, self._STOP):
            if self._worker_error is not None:
                continue                     # drop what was queued behind a failed write
            try:
                self._log(item[0], iteration=item[1])
            except BaseException as error:   # logging must never stop training
                self._give_up(error)

    def write(self, metrics: Mapping[str, float], *, iteration: int) -> None:
        if not is_rank0():
            return
        if not self.async_write:
            self._log(metrics, iteration=iteration)
            return
        with self._gate:
            if self._closing or self._closed or self._worker_error is not None:
                return
            if self._worker is None:
                try:
                    with _sdk_lock:          # a missing SDK is reported here, not on the worker
                        _ProcessRun.attach(self)
                except Exception as error:
                    self._give_up(error)
                    return
                self._inbox = SimpleQueue()
                self._worker = threading.Thread(target=self._drain, name="wm-wandb-metrics", daemon=True)
                self._worker.start()
            # a copy: the caller may release its reduction buffers at once
            self._inbox.put((dict(metrics), int(iteration)))

    def close(self) -> None:
        with self._gate:
            worker, first = self._worker, not self._closing
            self._closing = True
            if worker is not None and first:
                self._inbox.put(self._STOP)
        if worker is not None:
            worker.join()
            if self._worker_error is not None:
                log.warning("W&B metric worker stopped: "
                            f"{type(self._worker_error).__name__}: {self._worker_error}")
        super().close()


class WandbArtifactWriter(_RunClient):
    """Sample media into the shared run: images as they are, clips encoded to mp4 here (handing
    raw frames to the SDK would route them through its own, slower and fragile, encoder)."""

    def __init__(self, project: str, group: str | None = None, name: str | None = None,
                 mode: str | None = None, *, layout: str = "BCTHW", float_range: str = "minus_one_one",
                 fps: int = 16, frame_chunk_size: int = 8, grid_layout: Sequence[Any] | None = None,
                 grid_condition_keys: Sequence[Any] | None = None, grid_reference_key: Any | None = None,
                 grid_name: str = "grid", save_individual_artifacts: bool = True,
                 video_quality: int = 5) -> None:
        super().__init__(project=project, group=group, name=name, mode=mode)
        # the file writer's artifact builder (grids, per-sample clips) without its file output
        self._builder = ImageVideoArtifactWriter(
            layout=layout, float_range=float_range, fps=fps, frame_chunk_size=frame_chunk_size,
            video_quality=video_quality, grid_layout=grid_layout, grid_condition_keys=grid_condition_keys,
            grid_reference_key=grid_reference_key, grid_name=grid_name,
            save_individual_artifacts=save_individual_artifacts)
        for field in ("layout", "float_range", "fps", "frame_chunk_size", "grid_layout",
                      "grid_condition_keys", "grid_reference_key", "grid_name",
                      "save_individual_artifacts", "video_quality"):
            setattr(self, field, getattr(self._builder, field))

    def write(self, value: Any, *, output_dir: str, split: str, iteration: int, rank: int,
              sample_batch_index: int = 0) -> None:
        del output_dir, rank
        if not is_rank0():
            return
        sdk = self._initialize()
        if sdk is None:
            return
        payload: dict[str, Any] = {}
        for name, index, count, pixels in self._builder._artifacts(value):
            where = f"{split}/batch_{int(sample_batch_index):04d}/{name}"
            if count != 1:
                where += f"/{index:03d}"
            if pixels.shape[0] == 1:
                payload[where] = sdk.Image(pixels[0].numpy())
            else:
                clip = io.encode_video(pixels.numpy(), fps=self.fps, quality=self.video_quality)
                payload[where] = sdk.Video(clip, format="mp4")
        if payload:
            self._log(payload, iteration=int(iteration))
