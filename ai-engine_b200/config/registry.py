"""One registry from an architecture's name (config.json `architectures[0]`) to
its configuration class and model builder.

The reference matches substrings of the lower-cased name
(crates/ai-engine-runtime/src/config.rs:186-200); here the match is exact and
an unknown name is an error that lists what is registered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .base import ConfigError, read_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type            # has from_dict(dict) and to_dict()
    build_spec: Callable        # config -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable) -> None:
    """Add an architecture.  `config_cls.from_dict(raw)` parses its config.json;
    `build_spec(config)` returns the ModelSpec (layers from parts, run order,
    tensor names) that the engine builds and steps."""
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: dict) -> Architecture:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs:
        raise ConfigError("config.json: required key `architectures` must be a non-empty list")
    for a in archs:
        if a in _ARCHITECTURES:
            return _ARCHITECTURES[a]
    raise ConfigError(
        f"config.json: architecture {archs!r} is not registered "
        f"(registered: {', '.join(registered_architectures()) or 'none'})")


def load_config(path_or_dict):
    """(Architecture, typed config) from a model folder, a config.json or a dict."""
    raw = path_or_dict if isinstance(path_or_dict, dict) else read_json(path_or_dict)
    arch = resolve_architecture(raw)
    return arch, arch.config_cls.from_dict(raw)
