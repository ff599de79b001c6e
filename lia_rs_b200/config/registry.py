"""One registry from an architecture's name to its configuration class and model builder.

The reference dispatches on config.json's `model_type` with a `match`
(src/models/mod.rs:41-51) and fails with "unsupported model architecture"; here the table
is open: `register_architecture` adds an entry, and an architecture is found by the first
name in config.json's `architectures`, then by `model_type`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type          # has from_dict(raw) and to_dict()
    build: Callable             # build(config) -> models.decoder.ModelSpec


_ARCHITECTURES: dict = {}


def register_architecture(names, config_class, build) -> None:
    """Register one architecture under one or several names (architectures[] entries or
    model_type values)."""
    if isinstance(names, str):
        names = (names,)
    for name in names:
        _ARCHITECTURES[name] = Architecture(name, config_class, build)


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: dict) -> Architecture:
    """The registry entry that config.json (as a dict) names."""
    candidates = list(raw.get("architectures") or [])
    if raw.get("model_type"):
        candidates.append(raw["model_type"])
    for name in candidates:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise ConfigError(
        f"unsupported model architecture {candidates!r}; known: {known_architectures()}")
