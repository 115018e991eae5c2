"""The one registry from an architecture's name (``model_type`` in
config.json) to its typed configuration and its model description.

The reference has no registry object: each binary matches on ``model_type``
(infernum-examples/examples/generate.rs:266-291) against a list of supported
names (infernum-llama/src/config.rs:129,152-156).  Here an architecture is an
entry ``{parse_config, build_spec}``; everything else (loader, cache, step,
scheduler, tools) goes through ``resolve``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping

from .config.base import read_config_json
from .errors import UnsupportedModelError
from .parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]  # config.json dict -> typed config
    build_spec: Callable[[Any], ModelSpec]  # typed config -> model description


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec) -> Architecture:
    arch = Architecture(name, parse_config, build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def supported_architectures() -> List[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def resolve(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnsupportedModelError(
            f"model_type {name!r} is not supported; supported: {sorted(_ARCHITECTURES)}"
        ) from None


def resolve_config(config: Mapping[str, Any]):
    """(architecture, typed config) for a config.json dict; a missing
    ``model_type`` means "llama" as in the reference (config.rs:21-22)."""
    arch = resolve(config.get("model_type", "llama"))
    return arch, arch.parse_config(config)


def resolve_folder(folder: str):
    return resolve_config(read_config_json(folder))


def _ensure_builtin() -> None:
    if "llama" not in _ARCHITECTURES:
        from .models import llama  # noqa: F401  (registers itself)
