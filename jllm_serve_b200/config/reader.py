"""Typed getters over a parsed config.json.

The reference's getters return the default on a missing key *or* on a value of the wrong
type (src/main/java/org/robomiri/jllm/json/Json.java:406-435). Here a wrong type is an
error that names the key: a typo in a config should not silently become a default.
"""
from __future__ import annotations

import math
from typing import Any, Mapping

from .specs import ConfigError

_MISSING = object()


class ConfigReader:
    def __init__(self, values: Mapping[str, Any], where: str = "config.json"):
        if not isinstance(values, Mapping):
            raise ConfigError(f"{where} must hold a JSON object")
        self.values = values
        self.where = where

    def has(self, key: str) -> bool:
        return key in self.values and self.values[key] is not None

    def _get(self, key, default):
        v = self.values.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return _MISSING
        return v

    def integer(self, key: str, default=_MISSING) -> int:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)) or (isinstance(v, float) and v != int(v)):
            raise ConfigError(f"{self.where}: '{key}' must be an integer, got {v!r}")
        return int(v)

    def positive(self, key: str, default=_MISSING) -> int:
        """A required positive integer (Families.java:1126-1133)."""
        v = self.integer(key, default)
        if v is not None and v <= 0:
            raise ConfigError(f"{self.where}: '{key}' must be positive, got {v}")
        return v

    def number(self, key: str, default=_MISSING) -> float:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
            raise ConfigError(f"{self.where}: '{key}' must be a finite number, got {v!r}")
        return float(v)

    def boolean(self, key: str, default=_MISSING) -> bool:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default=_MISSING) -> str:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, got {v!r}")
        return v

    def int_list(self, key: str) -> tuple:
        """An integer or a list of integers (eos_token_id; Families.java:1099-1118). Missing = empty."""
        v = self.values.get(key)
        if v is None:
            return ()
        items = v if isinstance(v, list) else [v]
        for x in items:
            if isinstance(x, bool) or not isinstance(x, int):
                raise ConfigError(f"{self.where}: '{key}' must be an integer or a list of integers, got {v!r}")
        return tuple(items)

    def mapping(self, key: str):
        v = self.values.get(key)
        if v is None:
            return None
        if not isinstance(v, Mapping):
            raise ConfigError(f"{self.where}: '{key}' must be an object, got {v!r}")
        return ConfigReader(v, f"{self.where}:{key}")
