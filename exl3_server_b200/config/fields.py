"""Typed access to the keys of a config.json object.

Every architecture's configuration class reads its keys through a
``KeyReader``: a required key that is absent, a value of the wrong type, or a
value outside its allowed range raises ``ConfigError`` naming the key, in the
manner of the reference's ``"config.json: " + what()`` messages
(src/model.cpp:176-179).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration."""


_MISSING = object()


class KeyReader:
    """Reads keys of one JSON object and remembers which keys were used."""

    def __init__(self, obj: Dict[str, Any], where: str = "config.json"):
        if not isinstance(obj, dict):
            raise ConfigError(f"{where}: expected a JSON object")
        self.obj = obj
        self.where = where
        self.used: set = set()

    def has(self, key: str) -> bool:
        return key in self.obj and self.obj[key] is not None

    def raw(self, key: str, default: Any = _MISSING) -> Any:
        self.used.add(key)
        if key not in self.obj or self.obj[key] is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return self.obj[key]

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = None) -> Optional[int]:
        v = self.raw(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = False) -> Optional[float]:
        v = self.raw(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> Optional[bool]:
        v = self.raw(key, default)
        if v is None:
            return None
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> Optional[str]:
        v = self.raw(key, default)
        if v is None:
            return None
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {v!r}")
        return v

    def int_list(self, key: str, default: Any = _MISSING) -> List[int]:
        """An integer or a list of integers (``eos_token_id`` comes in both
        forms, src/model.cpp:108-114)."""
        v = self.raw(key, default)
        if v is None:
            return []
        if isinstance(v, int) and not isinstance(v, bool):
            return [v]
        if isinstance(v, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in v):
            return list(v)
        raise ConfigError(f"{self.where}: key '{key}' must be an integer or a list of integers, got {v!r}")


def read_config_json(model_dir: str) -> Dict[str, Any]:
    """Parses ``<model_dir>/config.json`` (``model_dir`` may also be the
    path of a file inside the folder, as in src/model.cpp:325-326)."""
    if os.path.isfile(model_dir):
        model_dir = os.path.dirname(model_dir) or "."
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            obj = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file")
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})")
    if not isinstance(obj, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return obj
