"""Lazy object configuration without external config libraries.

A configuration is a tree of :class:`ConfigNode` (mapping with attribute access) and
:class:`ListNode`.  ``LazyCall(T)(**kw)`` records a keyword call as
``{_target_: "dotted.path", **defaults_of_T, **kw}``; :func:`instantiate` builds the tree
bottom-up.  String values may reference other values with ``${a.b.c}`` and the
environment with ``${oc.env:NAME,default}``; ``???`` marks a value that must be supplied.
:func:`apply_overrides` implements the command-line grammar
(``a.b=1``, ``+a.b=x``, ``++a.b=x``, ``~a.b``, ``a={k:v,l:[1,2]}``, ``a=null``).

Resolved trees contain only YAML scalars, lists and mappings, so they round-trip through
``to_yaml``/``from_yaml`` — inference reads ``config.yaml`` back without importing recipes.

Parity: reference ``wm/infra/config.py:26-193`` (locate / LazyCall / instantiate) and the
override and interpolation behaviour it gets from hydra/omegaconf
(``wm/configs/compose.py:50-81``).
"""

from __future__ import annotations

import collections.abc as abc
import dataclasses
import enum
import importlib
import inspect
import os
import re
from collections.abc import Callable, Iterator, Sequence
from typing import Any, Generic, TypeVar

import yaml

__all__ = [
    "MISSING",
    "ConfigError",
    "ConfigNode",
    "LazyCall",
    "LazyDict",
    "ListNode",
    "apply_overrides",
    "from_yaml",
    "instantiate",
    "locate",
    "parse_override",
    "resolve",
    "to_container",
    "to_yaml",
]

MISSING = "???"
T = TypeVar("T")


class ConfigError(ValueError):
    """Raised for malformed overrides, missing values or bad interpolations."""


# --------------------------------------------------------------------------- tree
def _wrap(value: Any) -> Any:
    if isinstance(value, (ConfigNode, ListNode)):
        return value
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        node = ConfigNode({f.name: getattr(value, f.name) for f in dataclasses.fields(value)})
        object.__setattr__(node, "_object_type", type(value))
        return node
    if isinstance(value, abc.Mapping):
        return ConfigNode(value)
    if isinstance(value, (list, tuple)):
        return ListNode(value)
    if isinstance(value, enum.Enum):
        return value.value
    return value


class ConfigNode(dict):
    """Mapping node with attribute access. Children are wrapped on assignment."""

    _object_type: type | None = None

    def __init__(self, data: abc.Mapping | None = None, **kwargs: Any) -> None:
        super().__init__()
        object.__setattr__(self, "_object_type", None)
        for key, value in {**(dict(data) if data else {}), **kwargs}.items():
            self[key] = value

    def __setitem__(self, key: str, value: Any) -> None:
        super().__setitem__(str(key), _wrap(value))

    def __getattr__(self, key: str) -> Any:
        if key.startswith("__"):
            raise AttributeError(key)
        try:
            return self[key]
        except KeyError as error:
            raise AttributeError(key) from error

    def __setattr__(self, key: str, value: Any) -> None:
        self[key] = value

    def __delattr__(self, key: str) -> None:
        del self[key]

    def setdefault(self, key: str, default: Any = None) -> Any:  # type: ignore[override]
        if key not in self:
            self[key] = default
        return self[key]

    def update(self, *args: Any, **kwargs: Any) -> None:  # type: ignore[override]
        for key, value in dict(*args, **kwargs).items():
            self[key] = value

    def copy(self) -> ConfigNode:  # type: ignore[override]
        return _clone(self)

    def __deepcopy__(self, memo: dict) -> ConfigNode:
        return _clone(self)


class ListNode(list):
    def __init__(self, data: Sequence | None = None) -> None:
        super().__init__(_wrap(v) for v in (data or ()))

    def append(self, value: Any) -> None:
        super().append(_wrap(value))

    def __setitem__(self, index: Any, value: Any) -> None:
        super().__setitem__(index, _wrap(value))

    def __deepcopy__(self, memo: dict) -> ListNode:
        return _clone(self)


LazyDict = ConfigNode


def _clone(value: Any) -> Any:
    if isinstance(value, ConfigNode):
        out = ConfigNode({k: _clone(v) for k, v in value.items()})
        object.__setattr__(out, "_object_type", value._object_type)
        return out
    if isinstance(value, ListNode):
        return ListNode([_clone(v) for v in value])
    return value


def to_container(value: Any) -> Any:
    """Plain ``dict``/``list`` copy (tuples become lists, enums their values)."""
    if isinstance(value, abc.Mapping):
        return {str(k): to_container(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [to_container(v) for v in value]
    if isinstance(value, enum.Enum):
        return value.value
    return value


def to_yaml(value: Any) -> str:
    return yaml.safe_dump(to_container(value), sort_keys=False, default_flow_style=False)


def from_yaml(text: str) -> Any:
    return _wrap(yaml.safe_load(text))


# ------------------------------------------------------------------ interpolation
_INTERP = re.compile(r"\$\{([^${}]+)\}")


def _select(root: Any, path: str) -> Any:
    node = root
    for part in path.split("."):
        if isinstance(node, abc.Mapping):
            if part not in node:
                raise ConfigError(f"interpolation key {path!r} not found (at {part!r})")
            node = node[part]
        elif isinstance(node, list):
            node = node[int(part)]
        else:
            raise ConfigError(f"interpolation key {path!r} walks into a scalar at {part!r}")
    return node


def _evaluate(expression: str, root: Any, stack: tuple[str, ...]) -> Any:
    expression = expression.strip()
    if expression.startswith("oc.env:"):
        name, _, default = expression[len("oc.env:"):].partition(",")
        value = os.environ.get(name.strip())
        if value is None:
            if not _:
                raise ConfigError(f"environment variable {name!r} is not set")
            value = default.strip()
            return None if value == "null" else value
        return value
    if expression in stack:
        raise ConfigError(f"interpolation cycle through {expression!r}")
    return _resolve_value(_select(root, expression), root, (*stack, expression))


def _resolve_value(value: Any, root: Any, stack: tuple[str, ...] = ()) -> Any:
    if isinstance(value, str) and "${" in value:
        whole = _INTERP.fullmatch(value)
        if whole:
            return _clone(_evaluate(whole.group(1), root, stack))
        previous = None
        while previous != value and "${" in value:
            previous = value
            value = _INTERP.sub(lambda m: str(_evaluate(m.group(1), root, stack)), value)
        return value
    if isinstance(value, ConfigNode):
        out = ConfigNode()
        object.__setattr__(out, "_object_type", value._object_type)
        for key, child in value.items():
            out[key] = _resolve_value(child, root, stack)
        return out
    if isinstance(value, ListNode):
        return ListNode([_resolve_value(child, root, stack) for child in value])
    return value


def resolve(config: ConfigNode, *, throw_on_missing: bool = True) -> ConfigNode:
    """Return a copy with every interpolation replaced; optionally fail on ``???``."""
    out = _resolve_value(config, config)
    if throw_on_missing:
        missing = [path for path, value in _walk(out) if value == MISSING]
        if missing:
            raise ConfigError(f"missing mandatory values: {', '.join(missing)}")
    return out


def _walk(value: Any, prefix: str = "") -> Iterator[tuple[str, Any]]:
    if isinstance(value, abc.Mapping):
        for key, child in value.items():
            yield from _walk(child, f"{prefix}.{key}" if prefix else str(key))
    elif isinstance(value, list):
        for index, child in enumerate(value):
            yield from _walk(child, f"{prefix}.{index}")
    else:
        yield prefix, value


# ---------------------------------------------------------------------- overrides
_NUMBER = re.compile(r"[+-]?(\d+\.?\d*([eE][+-]?\d+)?|\.\d+([eE][+-]?\d+)?|inf|nan)")


class _ValueParser:
    """Recursive-descent parser for override values (scalars, lists, dicts)."""

    def __init__(self, text: str) -> None:
        self.text, self.pos = text, 0

    def parse(self) -> Any:
        value = self._value(top=True)
        self._space()
        if self.pos != len(self.text):
            raise ConfigError(f"trailing characters in override value {self.text!r}")
        return value

    def _space(self) -> None:
        while self.pos < len(self.text) and self.text[self.pos].isspace():
            self.pos += 1

    def _value(self, top: bool = False) -> Any:
        self._space()
        if self.pos >= len(self.text):
            return ""
        char = self.text[self.pos]
        if char == "[":
            return self._list()
        if char == "{":
            return self._dict()
        if char in "\"'":
            return self._quoted(char)
        return self._bare(top)

    def _quoted(self, quote: str) -> str:
        self.pos += 1
        out = []
        while self.pos < len(self.text) and self.text[self.pos] != quote:
            if self.text[self.pos] == "\\" and self.pos + 1 < len(self.text):
                self.pos += 1
            out.append(self.text[self.pos])
            self.pos += 1
        if self.pos >= len(self.text):
            raise ConfigError(f"unterminated quote in {self.text!r}")
        self.pos += 1
        return "".join(out)

    def _bare(self, top: bool) -> Any:
        start, depth = self.pos, 0
        while self.pos < len(self.text):
            char = self.text[self.pos]
            if self.text.startswith("${", self.pos):
                depth += 1
                self.pos += 2
                continue
            if depth and char == "}":
                depth -= 1
            elif not depth and not top and char in ",]}":
                break
            elif not depth and not top and char == ":" :
                break
            self.pos += 1
        return _scalar(self.text[start:self.pos].strip())

    def _list(self) -> list:
        self.pos += 1
        items: list[Any] = []
        while True:
            self._space()
            if self.pos >= len(self.text):
                raise ConfigError(f"unterminated list in {self.text!r}")
            if self.text[self.pos] == "]":
                self.pos += 1
                return items
            items.append(self._value())
            self._space()
            if self.pos < len(self.text) and self.text[self.pos] == ",":
                self.pos += 1

    def _dict(self) -> dict:
        self.pos += 1
        items: dict[str, Any] = {}
        while True:
            self._space()
            if self.pos >= len(self.text):
                raise ConfigError(f"unterminated dict in {self.text!r}")
            if self.text[self.pos] == "}":
                self.pos += 1
                return items
            key = self._value()
            self._space()
            if self.pos >= len(self.text) or self.text[self.pos] != ":":
                raise ConfigError(f"expected ':' after key {key!r} in {self.text!r}")
            self.pos += 1
            items[str(key)] = self._value()
            self._space()
            if self.pos < len(self.text) and self.text[self.pos] == ",":
                self.pos += 1


def _scalar(text: str) -> Any:
    lowered = text.lower()
    if lowered in ("null", "none", "~"):
        return None
    if lowered == "true":
        return True
    if lowered == "false":
        return False
    if _NUMBER.fullmatch(lowered):
        try:
            return int(text)
        except ValueError:
            return float(text)
    return text


@dataclasses.dataclass(frozen=True)
class Override:
    key: str
    value: Any = None
    kind: str = "set"  # set | add | force_add | delete


def parse_override(text: str) -> Override:
    if text.startswith("~"):
        key, _, _value = text[1:].partition("=")
        return Override(key.strip(), None, "delete")
    kind = "set"
    if text.startswith("++"):
        kind, text = "force_add", text[2:]
    elif text.startswith("+"):
        kind, text = "add", text[1:]
    if "=" not in text:
        raise ConfigError(f"override {text!r} is not of the form key=value")
    key, _, raw = text.partition("=")
    key = key.strip()
    if not key or not all(part for part in key.split(".")):
        raise ConfigError(f"bad override key in {text!r}")
    return Override(key, _ValueParser(raw).parse(), kind)


def apply_overrides(config: ConfigNode, overrides: Sequence[str | Override]) -> ConfigNode:
    """Apply overrides in place and return ``config``.

    ``key=value`` needs an existing key; ``+key=value`` needs a new key; ``++`` accepts
    both; ``~key`` deletes.  Mapping values merge into existing mapping nodes unless they
    carry their own ``_target_`` (then they replace the node).
    """
    for item in overrides:
        override = parse_override(item) if isinstance(item, str) else item
        *parents, leaf = override.key.split(".")
        node: Any = config
        for part in parents:
            if isinstance(node, list):
                node = node[int(part)]
                continue
            if part not in node:
                if override.kind == "set":
                    raise ConfigError(f"override {override.key!r}: no such key {part!r}")
                node[part] = ConfigNode()
            node = node[part]
        if override.kind == "delete":
            if leaf not in node:
                raise ConfigError(f"cannot delete missing key {override.key!r}")
            del node[leaf]
            continue
        if isinstance(node, list):
            node[int(leaf)] = override.value
            continue
        present = leaf in node
        if override.kind == "set" and not present:
            raise ConfigError(
                f"override {override.key!r}: key does not exist (use +{override.key}=...)")
        if override.kind == "add" and present:
            raise ConfigError(
                f"override +{override.key}: key already exists (use {override.key}=... or ++)")
        current = node.get(leaf)
        if (isinstance(current, ConfigNode) and isinstance(override.value, abc.Mapping)
                and "_target_" not in override.value):
            _merge(current, override.value)
        else:
            node[leaf] = override.value
    return config


def _merge(dest: ConfigNode, source: abc.Mapping) -> None:
    for key, value in source.items():
        if isinstance(dest.get(key), ConfigNode) and isinstance(value, abc.Mapping) \
                and "_target_" not in value:
            _merge(dest[key], value)
        else:
            dest[key] = value


# ------------------------------------------------------------------ lazy targets
def locate(name: str) -> Any:
    """Import the object named by a dotted path.

    Tries progressively shorter module prefixes; an ImportError raised *inside* a real
    module (a missing dependency) is propagated instead of being masked.
    """
    if not isinstance(name, str) or "." not in name or "<locals>" in name:
        raise ImportError(f"target must be an importable dotted path, got {name!r}")
    parts = name.split(".")
    for split in range(len(parts), 0, -1):
        module_name = ".".join(parts[:split])
        try:
            obj: Any = importlib.import_module(module_name)
        except ModuleNotFoundError as error:
            missing = error.name or ""
            if module_name != missing and not module_name.startswith(missing + "."):
                raise
            continue
        try:
            for attribute in parts[split:]:
                obj = getattr(obj, attribute)
        except AttributeError as error:
            raise ImportError(f"cannot locate target {name!r}") from error
        return obj
    raise ImportError(f"cannot import target {name!r}")


def _target_string(target: Any) -> str:
    module = getattr(target, "__module__", None)
    qualname = getattr(target, "__qualname__", None)
    if not isinstance(module, str) or not isinstance(qualname, str):
        raise TypeError(f"LazyCall target is not an importable callable: {target!r}")
    if module in {"__main__", "__mp_main__"} or "<locals>" in qualname or "<lambda>" in qualname:
        raise ValueError(f"LazyCall target is not importable: {module}.{qualname}")
    pieces = module.split(".")
    # Prefer the shortest package path that exports the same object.
    for end in range(1, len(pieces) + 1):
        candidate = f"{'.'.join(pieces[:end])}.{qualname}"
        try:
            if locate(candidate) is target:
                return candidate
        except ImportError:
            continue
    raise ValueError(f"LazyCall target {module}.{qualname} cannot be imported by dotted path")


def _signature_defaults(target: Callable[..., Any]) -> dict[str, Any]:
    if isinstance(target, type) and dataclasses.is_dataclass(target):
        # A ``default_factory`` shows up in the signature as an opaque sentinel: call it instead.
        defaults: dict[str, Any] = {}
        for field in dataclasses.fields(target):
            if not field.init:
                continue
            if field.default is not dataclasses.MISSING:
                defaults[field.name] = field.default
            elif field.default_factory is not dataclasses.MISSING:
                defaults[field.name] = field.default_factory()
        return defaults
    try:
        signature = inspect.signature(target)
    except (TypeError, ValueError):
        return {}
    kinds = (inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect.Parameter.KEYWORD_ONLY)
    return {
        name: parameter.default
        for name, parameter in signature.parameters.items()
        if parameter.default is not inspect.Parameter.empty and parameter.kind in kinds
    }


class LazyCall(Generic[T]):
    """``LazyCall(T)(**kw)`` → config node describing the call ``T(**kw)``."""

    def __init__(self, target: Callable[..., T] | str) -> None:
        if isinstance(target, str):
            resolved = locate(target)
            if not callable(resolved):
                raise TypeError(f"LazyCall target {target!r} is not callable")
            self._target, self._callable = target, resolved
        elif callable(target):
            self._target, self._callable = _target_string(target), target
        else:
            raise TypeError(f"LazyCall target must be an importable callable, got {target!r}")

    def __call__(self, **kwargs: Any) -> ConfigNode:
        parameters = _signature_defaults(self._callable)
        parameters.update(kwargs)
        node = ConfigNode({"_target_": self._target})
        for key, value in parameters.items():
            node[key] = value
        return node


def instantiate(cfg: Any, *args: Any, **kwargs: Any) -> Any:
    """Build the object tree described by ``cfg``.

    Keyword arguments given here override config keys and are passed through as they are
    (never instantiated).  ``_recursive_: false`` hands child configs to the target
    untouched.  Nodes that were created from a dataclass instance are rebuilt as that
    dataclass.
    """
    if isinstance(cfg, list):
        return [instantiate(value) for value in cfg]
    if isinstance(cfg, ConfigNode) and cfg._object_type is not None:
        return cfg._object_type(**{k: instantiate(v) for k, v in cfg.items()})
    if isinstance(cfg, abc.Mapping) and "_target_" in cfg:
        name = cfg["_target_"]
        if not isinstance(name, str):
            raise TypeError(f"_target_ must be an importable dotted string, got {name!r}")
        target = locate(name)
        if not callable(target):
            raise TypeError(f"_target_ {name!r} does not name a callable")
        recursive = cfg.get("_recursive_", True)
        values: dict[str, Any] = {}
        for key in cfg:
            if key in ("_target_", "_recursive_"):
                continue
            if key in kwargs:
                values[key] = kwargs[key]
            else:
                values[key] = instantiate(cfg[key]) if recursive else cfg[key]
        for key, value in kwargs.items():
            values.setdefault(key, value)
        return target(*args, **values)
    if isinstance(cfg, abc.Mapping):
        return {key: instantiate(value) for key, value in cfg.items()}
    return cfg
