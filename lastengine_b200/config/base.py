"""Typed reading of a model's config.json.

Every size and constant of a model comes from its config.json; code holds only
defaults for keys the architecture itself defines as optional.  The reference
reads its hyper-parameters the same way from GGUF metadata and stops with the
name of a missing key (src/dense.rs:52-77).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Sequence


class ConfigError(ValueError):
    """A config.json that cannot describe a model: names the key and the reason."""


_MISSING = object()


class KeyReader:
    """Reads typed values out of a parsed config.json and remembers which keys were used."""

    def __init__(self, raw: dict[str, Any], where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = raw
        self.where = where
        self.used: set[str] = set()

    def has(self, key: str) -> bool:
        return key in self.raw and self.raw[key] is not None

    def _get(self, keys: Sequence[str], default: Any) -> tuple[str, Any]:
        for k in keys:
            if self.has(k):
                self.used.add(k)
                return k, self.raw[k]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: missing required key '{keys[0]}'")
        return keys[0], default

    def integer(self, *keys: str, default: Any = _MISSING, minimum: int | None = None) -> int:
        k, v = self._get(keys, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: '{k}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: '{k}' must be >= {minimum}, got {v}")
        return v

    def number(self, *keys: str, default: Any = _MISSING) -> float:
        k, v = self._get(keys, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{k}' must be a number, got {v!r}")
        return float(v)

    def boolean(self, *keys: str, default: Any = _MISSING) -> bool:
        k, v = self._get(keys, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{k}' must be true or false, got {v!r}")
        return v

    def string(self, *keys: str, default: Any = _MISSING) -> str:
        k, v = self._get(keys, default)
        if v is not None and not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{k}' must be a string, got {v!r}")
        return v

    def array(self, *keys: str, default: Any = _MISSING, item: Callable[[Any], bool] | None = None) -> list:
        k, v = self._get(keys, default)
        if v is None:
            return v
        if not isinstance(v, list):
            raise ConfigError(f"{self.where}: '{k}' must be an array, got {v!r}")
        if item is not None:
            for i, e in enumerate(v):
                if not item(e):
                    raise ConfigError(f"{self.where}: '{k}'[{i}] has an invalid value {e!r}")
        return list(v)


def read_config_json(path: str) -> dict[str, Any]:
    """Parses DIR/config.json (or a path to the file itself)."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None


def architecture_name(raw: dict[str, Any]) -> str:
    """The name the registry is asked for: `architectures[0]`, else `model_type`."""
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = raw.get("model_type")
    if isinstance(mt, str):
        return mt
    raise ConfigError("config.json: neither 'architectures' nor 'model_type' names the model")
