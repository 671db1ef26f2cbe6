from .base import (PartSpec, KVSpec, StateSpec, Runtime, StepContext, UnitCache, Part, Norm, PositionEncoding,
                   Mixer, FeedForward, Block)
from .registry import (register_mixer, register_feed_forward, register_norm, register_position, register_block,
                       register_embedding, register_head, build_part, kinds)
from . import norm, rotary, attention, mlp, block, embedding  # noqa: F401  (register the built-in kinds)

__all__ = ["PartSpec", "KVSpec", "StateSpec", "Runtime", "StepContext", "UnitCache", "Part", "Norm",
           "PositionEncoding", "Mixer", "FeedForward", "Block", "register_mixer", "register_feed_forward",
           "register_norm", "register_position", "register_block", "register_embedding", "register_head",
           "build_part", "kinds"]
