"""Trainer callbacks."""

from .base import Callback, CallbackGroup
from .grad_clip import GradClip
from .grad_monitor import GradClipMonitor
from .media import ImageVideoArtifactWriter
from .metrics import LoguruMetricSink, MetricSink, ScalarMetricCallback
from .sampling import ArtifactWriter, ArtifactWriterGroup, PeriodicSampleCallback
from .wandb import WandbArtifactWriter, WandbMetricSink

__all__ = ["ArtifactWriter", "ArtifactWriterGroup", "Callback", "CallbackGroup", "GradClip",
           "GradClipMonitor", "ImageVideoArtifactWriter", "LoguruMetricSink", "MetricSink",
           "PeriodicSampleCallback", "ScalarMetricCallback", "WandbArtifactWriter", "WandbMetricSink"]
