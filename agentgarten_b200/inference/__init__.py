"""Inference: artifact IO, serving preparation, streaming."""
