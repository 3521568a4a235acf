"""Base class of networks that the parallel engine shards.

Parity: reference ``wm/infra/parallel.py:97-119`` (``ParallelNetwork``).
"""

from __future__ import annotations

from typing import ClassVar

from torch import nn

__all__ = ["ParallelNetwork"]


class ParallelNetwork(nn.Module):
    """A layered network: every entry of ``layers`` is one sharding unit and one
    activation-recompute unit."""

    layers: nn.ModuleList
    # Root methods besides ``forward`` that run the layers.
    fsdp_entry_points: ClassVar[tuple[str, ...]] = ()

    def fsdp_units(self) -> tuple[nn.Module, ...]:
        """Modules outside ``layers`` that are sharded as units of their own."""
        return ()

    def enable_context_parallel(self, mesh) -> None:
        """Networks that do not split tokens across ranks ignore the mesh."""
        del mesh

    def initialize_after_materialization(self) -> None:
        """Initialise parameters that no checkpoint provides, after ``to_empty``."""
        return
