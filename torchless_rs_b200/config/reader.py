"""Typed access to the keys of a config.json dictionary.

The reference reads the same keys one by one and leaves a field empty when the
key is absent or has another type (src/loader/formats/safetensors.rs:701-765);
here an absent required key or a wrong type is an error that names the key.
"""
from __future__ import annotations

import json
import os
from typing import Any

from .errors import ConfigError

_MISSING = object()


class KeyReader:
    """Reads typed values out of one JSON object and remembers which keys were used."""

    def __init__(self, data: dict, where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.data = data
        self.where = where

    def _get(self, key: str, default: Any):
        v = self.data.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return _MISSING
        return v

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = 1) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = True) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {v}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {v!r}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {v!r}")
        return v

    def list_of(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, list):
            raise ConfigError(f"{self.where}: key '{key}' must be a list, got {v!r}")
        return v


def read_config_json(model_dir: str) -> dict:
    """The config.json that lies beside the weights
    (src/loader/formats/safetensors.rs:675-698 looks in the same place)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
