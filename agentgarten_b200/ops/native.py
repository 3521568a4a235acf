"""Loader for the in-tree CUDA extension ``agentgarten_b200/_C*.so``.

The extension is built by ``python -m agentgarten_b200.build`` (nvcc, sm_100a only) and
lives inside the package directory.  ``use(tensor)`` tells an operator whether the CUDA
kernels apply to a tensor; on a CUDA device without the extension it raises, so a GPU run
can never silently fall back to library kernels.
"""

from __future__ import annotations

import importlib
import os
import threading
from typing import Any

import torch

__all__ = ["available", "ext", "launches", "require", "use"]

_lock = threading.Lock()
_ext: Any = None
_error: BaseException | None = None
_tried = False
_launches = 0


def _load() -> None:
    global _ext, _error, _tried
    with _lock:
        if _tried:
            return
        _tried = True
        if os.environ.get("AGB200_DISABLE_NATIVE") == "1":
            _error = RuntimeError("disabled by AGB200_DISABLE_NATIVE=1")
            return
        try:
            _ext = importlib.import_module("agentgarten_b200._C")
        except BaseException as error:  # ImportError, OSError (missing libs)
            _error = error


def available() -> bool:
    _load()
    return _ext is not None


def ext() -> Any:
    _load()
    if _ext is None:
        raise RuntimeError(
            "agentgarten_b200._C is not built or failed to load "
            f"({_error!r}); run `python -m agentgarten_b200.build`")
    return _ext


def require() -> Any:
    return ext()


def use(*tensors: torch.Tensor, dtypes: tuple[torch.dtype, ...] = (torch.bfloat16,)) -> bool:
    """True when the CUDA kernels should handle these tensors."""
    first = tensors[0]
    if not first.is_cuda:
        return False
    if os.environ.get("AGB200_DISABLE_NATIVE") == "1":
        return False
    if first.dtype not in dtypes:
        return False
    ext()  # raises loudly on a GPU box without the extension
    return True


def count(n: int = 1) -> None:
    """Bookkeeping of kernel launches issued through this package."""
    global _launches
    _launches += n


def launches() -> int:
    return _launches
