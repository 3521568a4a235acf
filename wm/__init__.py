"""Import alias: ``wm.<module>`` resolves to the matching ``agentgarten_b200`` module.

Configuration files, checkpoints' ``config.yaml`` and user code written against the ``wm``
package keep working: ``wm.models.diffusion.DiffusionModel`` is the same object as
``agentgarten_b200.models.diffusion.DiffusionModel``.  A few modules live elsewhere in this
package; ``_RELOCATED`` lists them.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

from agentgarten_b200 import __version__

_RELOCATED = {
    "wm.infra.parallel": "agentgarten_b200.parallel.engine",
    "wm.infra.log": "agentgarten_b200.utils.log",
    "wm.infra.io": "agentgarten_b200.utils.io",
    "wm.infra.utils": "agentgarten_b200.utils.misc",
    "wm.kernels": "agentgarten_b200.ops.kernels",
    "wm.kernels.gen_layer": "agentgarten_b200.ops.kernels.gen_layer",
    "wm.kernels.stream_cache": "agentgarten_b200.ops.kernels.stream_cache",
    "wm.kernels.attention_jvp": "agentgarten_b200.ops.kernels.attention_jvp",
}


def _target(name: str) -> str:
    if name in _RELOCATED:
        return _RELOCATED[name]
    return "agentgarten_b200" + name[len("wm"):]


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str) -> None:
        self.target = target

    def create_module(self, spec):
        module = importlib.import_module(self.target)
        return module

    def exec_module(self, module) -> None:  # already executed under its real name
        return


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("wm."):
            return None
        real = _target(fullname)
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real),
                                               is_package=found.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__all__ = ["__version__"]
