"""Typed reading of a model folder's ``config.json``.

A configuration class lists its keys once, as dataclass fields, and reads them
with the typed getters below.  Every error names the key that caused it.  The
reference keeps the same information in ``struct HParams`` (core/model.h:34-82)
and fills it in ``load_hparams`` (core/model.cpp:504-567) with typed getters
that tolerate the stored integer width (core/gguf_util.cpp:11-87).
"""
from __future__ import annotations

import json
import math
import os
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


_MISSING = object()


class ConfigReader:
    """Typed getters over a parsed config.json that remember which keys were read."""

    def __init__(self, data: Mapping[str, Any], where: str = "config.json"):
        if not isinstance(data, Mapping):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.data = data
        self.where = where
        self.read_keys: set[str] = set()

    def _raw(self, key: str, default: Any = _MISSING) -> Any:
        self.read_keys.add(key)
        if key not in self.data or self.data[key] is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return self.data[key]

    def has(self, key: str) -> bool:
        return key in self.data and self.data[key] is not None

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = None) -> int:
        v = self._raw(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {v!r}")
        v = int(v)
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = False) -> float:
        v = self._raw(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
            raise ConfigError(f"{self.where}: key '{key}' must be a finite number, got {v!r}")
        if positive and not v > 0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {v}")
        return float(v)

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self._raw(key, default)
        if v is default and default is not _MISSING:
            return v
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self._raw(key, default)
        if v is default and default is not _MISSING:
            return v
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {v!r}")
        return v

    def int_list(self, key: str, default: Any = _MISSING) -> list[int]:
        """An integer or a list of integers (``eos_token_id`` comes in both forms)."""
        v = self._raw(key, default)
        if v is default and default is not _MISSING:
            return v
        items = v if isinstance(v, list) else [v]
        out = []
        for x in items:
            if isinstance(x, bool) or not isinstance(x, int):
                raise ConfigError(f"{self.where}: key '{key}' must hold integers, got {x!r}")
            out.append(int(x))
        return out

    def mapping(self, key: str, default: Any = _MISSING) -> Any:
        v = self._raw(key, default)
        if v is default and default is not _MISSING:
            return v
        if not isinstance(v, Mapping):
            raise ConfigError(f"{self.where}: key '{key}' must be an object, got {v!r}")
        return v


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            data = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return data


class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses are dataclasses; they implement ``from_reader`` (typed reads and
    validation) and ``to_dict`` (the config.json that the random-weights mode
    writes; reading it back gives an equal object).
    """

    architecture: str = ""

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "ModelConfig":
        raise NotImplementedError

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config") -> "ModelConfig":
        return cls.from_reader(ConfigReader(data, where))

    def to_dict(self) -> dict:
        raise NotImplementedError
