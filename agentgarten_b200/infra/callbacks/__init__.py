"""Trainer callbacks."""

from .base import Callback, CallbackGroup
from .grad_clip import GradClip
from .grad_monitor import GradClipMonitor
from .metrics import LoguruMetricSink, MetricSink, ScalarMetricCallback

__all__ = ["Callback", "CallbackGroup", "GradClip", "GradClipMonitor", "LoguruMetricSink",
           "MetricSink", "ScalarMetricCallback"]
