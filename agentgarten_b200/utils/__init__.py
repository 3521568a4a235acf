"""Host-side utilities: logging, atomic IO, tensor-tree helpers."""

from . import io, log, misc

__all__ = ["io", "log", "misc"]
