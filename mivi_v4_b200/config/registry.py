"""One registry from an architecture's name (config.json ``architectures[0]``)
to its typed configuration and to the function that describes its model.

The reference's model crate never dispatches on an architecture name: it infers
layer kinds from tensor names (crates/mivi-model/src/loader.rs:157-174).  A
library that is meant to take further architectures needs the dispatch, so it
lives here, in one table.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[dict], Any]     # config.json dict -> typed config
    describe: Callable[[Any], Any]              # typed config -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict: Callable[[dict], Any],
                          describe: Callable[[Any], Any], *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, describe)


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_for(config_dict: dict) -> Architecture:
    """The entry for config.json's ``architectures[0]``."""
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(
            "config.json has no 'architectures' list; known architectures: "
            + ", ".join(known_architectures()))
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; known architectures: " + ", ".join(known_architectures()))
    return _ARCHITECTURES[name]
