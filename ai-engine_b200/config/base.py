"""Typed reading of config.json values.

Every size and constant of a model comes from its config.json through these
helpers; a wrong type or a missing required key is a `ConfigError` that names
the key.
"""
from __future__ import annotations

import json
import os


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


_MISSING = object()


def read_json(path: str) -> dict:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"config.json parse: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError("config.json must hold a JSON object")
    return raw


def get_int(raw: dict, key: str, default=_MISSING, minimum: int = 1) -> int:
    v = raw.get(key, None)
    if v is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key `{key}` is missing")
        return default
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: `{key}` must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: `{key}` must be >= {minimum}, got {v}")
    return v


def get_float(raw: dict, key: str, default=_MISSING) -> float:
    v = raw.get(key, None)
    if v is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key `{key}` is missing")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: `{key}` must be a number, got {v!r}")
    return float(v)


def get_bool(raw: dict, key: str, default: bool) -> bool:
    v = raw.get(key, None)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: `{key}` must be true or false, got {v!r}")
    return v
