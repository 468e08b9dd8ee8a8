"""The one registry from an architecture's name (config.json's ``architectures[0]``) to
its typed configuration and the function that lays out its model.

The reference tells families apart by a string match on the GGUF architecture
(crates/bc-infer/src/model.rs:45-48); here the same decision is a table that tests and
later architectures add rows to.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from ..config.errors import ConfigError
from ..parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed configuration
    model_spec: Callable[[Any], ModelSpec]             # typed configuration -> layout of parts


_architectures: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable, model_spec: Callable) -> None:
    _architectures[name] = Architecture(name, parse_config, model_spec)


def unregister_architecture(name: str) -> None:
    _architectures.pop(name, None)


def architecture_names():
    return sorted(_architectures)


def resolve(config: Mapping[str, Any]) -> Architecture:
    """The architecture a config.json names."""
    archs = config.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    if archs[0] not in _architectures:
        raise ConfigError(f"config.json: architecture {archs[0]!r} is not supported (known: {architecture_names()})")
    return _architectures[archs[0]]
