"""Typed reading of an architecture's own config.json keys.

The reference reads every hyperparameter through typed getters whose errors name
the missing key (crates/kf-arch/src/hparams.rs:202-261, `Keys::req`).  This module
is the same idea over a config.json dictionary: a reader that hands out typed
values, remembers which keys were read, and raises `ConfigError` naming the key.
"""
from __future__ import annotations

import json
import os
from typing import Any, Sequence


class ConfigError(ValueError):
    """A config.json that cannot describe a model: missing key, wrong type, bad value."""


_MISSING = object()


class KeyReader:
    """Typed getters over one config.json dictionary."""

    def __init__(self, raw: dict, where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: expected a JSON object, found {type(raw).__name__}")
        self.raw = raw
        self.where = where
        self.read: set[str] = set()

    def _get(self, key: str, default: Any) -> Any:
        self.read.add(key)
        if key in self.raw and self.raw[key] is not None:
            return self.raw[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: required key '{key}' is missing")
        return default

    def int(self, key: str, default: Any = _MISSING, *, min: int | None = None) -> int:
        v = self._get(key, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, found {v!r}")
        if min is not None and v < min:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {min}, found {v}")
        return v

    def float(self, key: str, default: Any = _MISSING) -> float:
        v = self._get(key, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, found {v!r}")
        return float(v)

    def bool(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, found {v!r}")
        return v

    def str(self, key: str, default: Any = _MISSING, *, choices: Sequence[str] | None = None) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, found {v!r}")
        if choices is not None and v not in choices:
            raise ConfigError(f"{self.where}: key '{key}' is {v!r}, expected one of {list(choices)}")
        return v

    def list(self, key: str, default: Any = _MISSING) -> list | None:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, list):
            raise ConfigError(f"{self.where}: key '{key}' must be a list, found {v!r}")
        return v


def read_config_json(path: str) -> dict:
    """The dictionary in `path` (a config.json, or a folder that holds one)."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def architecture_name(raw: dict, where: str = "config.json") -> str:
    """The model class a config.json asks for: `architectures[0]`."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: required key 'architectures' must be a non-empty list of names")
    return archs[0]
