"""Training runtime: configuration, trainer, callbacks, checkpoints, process groups.

Four modules that user code reaches as ``wm.infra.<name>`` live elsewhere in this package (the
logging, file and tree helpers under ``utils``, the placement engine under ``parallel``).  The
import alias resolves ``import wm.infra.io``; the names below make ``from wm.infra import io``
(and ``log``, ``utils``, ``parallel``) resolve as well, on first use.
"""

from __future__ import annotations

import importlib

_ELSEWHERE = {
    "io": "agentgarten_b200.utils.io",
    "log": "agentgarten_b200.utils.log",
    "utils": "agentgarten_b200.utils.misc",
    "parallel": "agentgarten_b200.parallel.engine",
}


def __getattr__(name: str):
    target = _ELSEWHERE.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    module = importlib.import_module(target)
    globals()[name] = module
    return module
