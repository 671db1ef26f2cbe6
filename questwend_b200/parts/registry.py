"""Registries of part kinds: name -> class.  A plan names kinds; ``build_part`` makes the objects."""
from __future__ import annotations

from .base import PartSpec, Runtime

_REGISTRIES: dict[str, dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str, cls: type, replace: bool = False):
    reg = _REGISTRIES[family]
    if kind in reg and not replace and reg[kind] is not cls:
        raise ValueError(f"{family} kind '{kind}' is already registered")
    reg[kind] = cls
    return cls


def register_mixer(kind, cls, replace=False):
    return _register("mixer", kind, cls, replace)


def register_feed_forward(kind, cls, replace=False):
    return _register("feed_forward", kind, cls, replace)


def register_norm(kind, cls, replace=False):
    return _register("norm", kind, cls, replace)


def register_position(kind, cls, replace=False):
    return _register("position", kind, cls, replace)


def register_block(kind, cls, replace=False):
    return _register("block", kind, cls, replace)


def register_embedding(kind, cls, replace=False):
    return _register("embedding", kind, cls, replace)


def register_head(kind, cls, replace=False):
    return _register("head", kind, cls, replace)


def kinds(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])


def build_part(family: str, spec: PartSpec, runtime: Runtime, **extra):
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise KeyError(f"unknown {family} kind '{spec.kind}'; registered: {', '.join(sorted(reg)) or '(none)'}")
    return reg[spec.kind](spec, runtime, **extra)
