"""One registry from an architecture's name (config.json ``model_type``) to its model.

An entry names the typed configuration class and a ``describe`` function that turns a
configuration into a ``ModelSpec``: plain data that lists, layer by layer, which parts
(mixer, feed-forward, norm, position encoding, block arrangement) the model is made of
and with which constants. Entries are import paths resolved on first use, like the
reference's registry (src/mlx_one/core/registry.py:11-116), so that naming an
architecture imports nothing until it is asked for.
"""

from __future__ import annotations

import importlib
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .base import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(mapping) and to_dict()
    describe: Callable[[Any], Any]         # configuration -> parts.spec.ModelSpec


_BUILTIN = {
    "lfm2": "mlx_one_b200.architectures.lfm2:ARCHITECTURE",
}
_REGISTERED: dict[str, Architecture] = {}


def register_architecture(architecture: Architecture, *, replace: bool = False) -> None:
    if not replace and (architecture.name in _REGISTERED or architecture.name in _BUILTIN):
        raise ValueError(f"architecture {architecture.name!r} is already registered")
    _REGISTERED[architecture.name] = architecture


def unregister_architecture(name: str) -> None:
    _REGISTERED.pop(name, None)


def architecture_names() -> tuple[str, ...]:
    return tuple(sorted(set(_BUILTIN) | set(_REGISTERED)))


def get_architecture(name: str) -> Architecture:
    if name in _REGISTERED:
        return _REGISTERED[name]
    if name in _BUILTIN:
        module_name, _, attribute = _BUILTIN[name].partition(":")
        entry = getattr(importlib.import_module(module_name), attribute)
        _REGISTERED[name] = entry
        return entry
    raise ConfigError(f"unknown architecture {name!r}; known: {', '.join(architecture_names())}")


def read_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """config.json of a model folder -> (registry entry, typed configuration)."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    data = json.loads(path.read_text())
    if "model_type" not in data:
        raise ConfigError(f"{path} has no model_type")
    entry = get_architecture(data["model_type"])
    return entry, entry.config_class.from_dict(data)
