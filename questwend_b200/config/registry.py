"""The one registry from an architecture's name to its model.

The reference maps ``general.architecture`` to an enum with an if-chain and
throws on an unknown name (core/model.cpp:30-37, 508-512).  Here an
architecture is an entry with the name that ``config.json`` carries in
``architectures[0]``, its configuration class, and a function that turns a
configuration into a model plan (the list of layers, the parts each is made
of, and the order they run in).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Mapping, Any

from .base import ConfigError, ConfigReader, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    plan: Callable[[ModelConfig], Any]      # ModelConfig -> engine.plan.ModelPlan


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, plan: Callable[[ModelConfig], Any],
                          replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    arch = Architecture(name, config_class, plan)
    _ARCHITECTURES[name] = arch
    return arch


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{name}'; registered: {', '.join(architectures()) or '(none)'}"
        ) from None


def architecture_name(data: Mapping[str, Any], where: str = "config.json") -> str:
    archs = data.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: key 'architectures' must be a list with one name, got {archs!r}")
    return archs[0]


def config_from_dict(data: Mapping[str, Any], where: str = "config.json") -> ModelConfig:
    arch = get_architecture(architecture_name(data, where))
    cfg = arch.config_class.from_reader(ConfigReader(data, where))
    return cfg


def load_config(model_dir: str) -> ModelConfig:
    import os
    data = read_config_json(model_dir)
    return config_from_dict(data, os.path.join(model_dir, "config.json"))
