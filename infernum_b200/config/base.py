"""Helpers shared by typed model configurations.

A configuration class is a frozen dataclass whose fields are exactly the
``config.json`` keys of its architecture.  ``read_config_json`` loads the file
and ``Field`` helpers below turn loose JSON values into checked Python values,
each failure naming the key at fault.
"""

from __future__ import annotations

import json
import os
from typing import Any, Mapping

from ..errors import ConfigError

_MISSING = object()


def read_config_json(path: str) -> dict:
    """Read ``config.json`` from a file path or from a model folder."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            data = json.load(fh)
    except FileNotFoundError as exc:
        raise ConfigError(f"no config.json at {path}") from exc
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return data


def take_int(d: Mapping[str, Any], key: str, default: Any = _MISSING, minimum: int = 1) -> int:
    value = d.get(key, _MISSING)
    if value is _MISSING or value is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {value}")
    return value


def take_float(d: Mapping[str, Any], key: str, default: Any = _MISSING) -> float:
    value = d.get(key, _MISSING)
    if value is _MISSING or value is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {value!r}")
    return float(value)


def take_bool(d: Mapping[str, Any], key: str, default: bool) -> bool:
    value = d.get(key, _MISSING)
    if value is _MISSING or value is None:
        return default
    if not isinstance(value, bool):
        raise ConfigError(f"config.json: '{key}' must be true or false, got {value!r}")
    return value


def take_int_or_first(d: Mapping[str, Any], key: str, default: int) -> int:
    """A scalar, or the first element of a list (the reference reads
    ``eos_token_id`` this way: infernum/src/serde_helpers.rs:14-31)."""
    value = d.get(key, _MISSING)
    if value is _MISSING or value is None:
        return default
    if isinstance(value, list):
        if not value:
            raise ConfigError(f"config.json: '{key}' is an empty list")
        value = value[0]
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: '{key}' must be an integer or a list of them")
    return value
