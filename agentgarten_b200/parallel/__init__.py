"""Parallel runtime: meshes, sharded-parameter engine, context and tensor parallelism,
peer-memory (NVLink) collectives."""

from .network import ParallelNetwork

__all__ = ["ParallelNetwork"]
