"""Stand-in for the ``omegaconf`` package, which is absent from the offline image.

Only what the reference package touches at import time and on the directly constructed
(config-free) benchmark path is provided: ``DictConfig`` / ``ListConfig`` containers with
attribute access and an ``OmegaConf`` namespace with the handful of helpers those modules
name.  Interpolation (``${...}``) is not implemented; the benchmark arm builds its objects
directly and never resolves a recipe tree.
"""

from __future__ import annotations

import types
from typing import Any

__all__ = ["DictConfig", "ListConfig", "OmegaConf", "MISSING"]
__version__ = "0.0-standin"

MISSING = "???"


def _wrap(value: Any) -> Any:
    if isinstance(value, (DictConfig, ListConfig)):
        return value
    if isinstance(value, dict):
        return DictConfig(value)
    if isinstance(value, (list, tuple)):
        return ListConfig(value)
    return value


class DictConfig(dict):
    def __init__(self, content: Any = None, flags: Any = None, **_: Any) -> None:
        super().__init__()
        object.__setattr__(self, "_metadata", types.SimpleNamespace(object_type=dict))
        for key, value in dict(content or {}).items():
            dict.__setitem__(self, key, _wrap(value))

    def __getattr__(self, name: str) -> Any:
        try:
            return self[name]
        except KeyError as error:
            raise AttributeError(name) from error

    def __setattr__(self, name: str, value: Any) -> None:
        self[name] = value

    def __setitem__(self, key: Any, value: Any) -> None:
        dict.__setitem__(self, key, _wrap(value))


class ListConfig(list):
    def __init__(self, content: Any = None, flags: Any = None, **_: Any) -> None:
        super().__init__(_wrap(value) for value in (content or ()))


def _plain(value: Any) -> Any:
    if isinstance(value, dict):
        return {key: _plain(item) for key, item in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(item) for item in value]
    return value


class OmegaConf:
    @staticmethod
    def create(content: Any = None, flags: Any = None) -> Any:
        return _wrap(content if content is not None else {})

    @staticmethod
    def to_container(config: Any, resolve: bool = False, **_: Any) -> Any:
        return _plain(config)

    @staticmethod
    def to_object(config: Any) -> Any:
        return _plain(config)

    @staticmethod
    def to_yaml(config: Any, resolve: bool = False, sort_keys: bool = False) -> str:
        import yaml

        return yaml.safe_dump(_plain(config), sort_keys=sort_keys)

    @staticmethod
    def is_config(value: Any) -> bool:
        return isinstance(value, (DictConfig, ListConfig))

    @staticmethod
    def resolve(config: Any) -> None:
        return None

    @staticmethod
    def register_new_resolver(*_: Any, **__: Any) -> None:
        return None

    @staticmethod
    def has_resolver(name: str) -> bool:
        return True

    @staticmethod
    def set_struct(config: Any, value: bool) -> None:
        return None
