"""One registry from an architecture's name to the code that knows it.

An :class:`Architecture` holds two callables: ``parse`` turns the dict read
from ``config.json`` into the architecture's typed configuration object, and
``build_spec`` turns that object into an architecture-neutral
:class:`~zedinfer_b200.config.spec.ModelSpec`.  The reference selects the model
with an ``if (model_type == ...)`` chain that throws ``Unsupported model type``
(src/frontend/models/base.cpp:419-463); here the chain is a table, so adding an
architecture means adding one file that calls :func:`register_architecture`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Tuple

from .spec import ModelSpec


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


@dataclass(frozen=True)
class Architecture:
    name: str
    model_types: Tuple[str, ...]
    parse: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, *, model_types: Tuple[str, ...] = (),
                          parse: Callable[[Mapping[str, Any]], Any],
                          build_spec: Callable[[Any], ModelSpec]) -> Architecture:
    arch = Architecture(name, tuple(model_types), parse, build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def supported_architectures() -> Tuple[str, ...]:
    _load_builtin()
    return tuple(sorted(_ARCHITECTURES))


def _load_builtin() -> None:
    # Importing the package registers every architecture that ships with it.
    from .. import models  # noqa: F401


def resolve_architecture(raw: Mapping[str, Any]) -> Architecture:
    """Pick the architecture for a config dict: ``architectures[0]``, else ``model_type``."""
    _load_builtin()
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    model_type = raw.get("model_type")
    if model_type is not None:
        for arch in _ARCHITECTURES.values():
            if model_type in arch.model_types:
                return arch
    raise ConfigError(
        f"Unsupported model: architectures={list(names)!r}, model_type={model_type!r}; "
        f"supported architectures: {', '.join(sorted(_ARCHITECTURES))}")


def read_config_json(model_dir: str) -> Dict[str, Any]:
    """The JSON object of ``model_dir/config.json``; ``model_dir`` may also name the JSON file itself."""
    path = model_dir if os.path.isfile(model_dir) else os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"Failed to open config file: {path}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return raw


def load_model_config(model_dir: str):
    """Read ``config.json`` → (architecture, typed config, ModelSpec)."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    cfg = arch.parse(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    return arch, cfg, spec
