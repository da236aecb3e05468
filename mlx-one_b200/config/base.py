"""Helpers shared by typed architecture configurations.

A configuration class is a frozen dataclass whose fields are the architecture's own
config.json keys. It checks every value when it is made and raises ``ConfigError``
with the key's name, as the reference does (src/mlx_one/core/config.py:10-26).
"""

from __future__ import annotations

import math
from typing import Any, Mapping


class ConfigError(ValueError):
    """config.json cannot describe a model that this engine can run."""


def positive(name: str, value: Any) -> None:
    bad = isinstance(value, bool) or not isinstance(value, (int, float))
    if bad or not math.isfinite(value) or value <= 0:
        raise ConfigError(f"{name} must be positive, got {value!r}")


def positive_int(name: str, value: Any) -> None:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"{name} must be a positive integer, got {value!r}")


def divisible(name: str, value: int, by_name: str, by: int) -> None:
    positive_int(name, value)
    positive_int(by_name, by)
    if value % by:
        raise ConfigError(f"{name} ({value}) must be divisible by {by_name} ({by})")


def boolean(name: str, value: Any) -> None:
    if not isinstance(value, bool):
        raise ConfigError(f"{name} must be a boolean, got {value!r}")


def unknown_keys(data: Mapping[str, Any], known: set[str]) -> dict[str, Any]:
    """Keys of config.json that the configuration class has no field for."""
    return {key: value for key, value in data.items() if key not in known}
