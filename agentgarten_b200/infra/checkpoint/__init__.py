"""Checkpointing: DCP tensors, sidecars, restore planning."""

from .checkpointer import DistributedCheckpointer, LoadResult

__all__ = ["DistributedCheckpointer", "LoadResult"]
