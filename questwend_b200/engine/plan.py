"""A model as data: which parts each layer is made of and the order the layers run in.

An architecture's plan function turns its configuration into a ``ModelPlan``.
``layers`` describes each layer by the kinds and parameters of its parts, so
one model can mix different mixers and feed-forwards.  ``schedule`` is the order
of execution: a list of ``Run`` entries.  An entry may name a layer that another
entry names too (the layer's weights are used twice; each run has a cache of its
own), and it may set ``cache_of`` to an earlier entry to read that run's cache
instead of owning one.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec                      # the arrangement; its prefix is the layer's tensor-name prefix
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec                       # the norm used inside the block
    position: PartSpec | None = None     # the mixer's position encoding


@dataclass(frozen=True)
class Run:
    layer: int                           # index into ModelPlan.layers
    cache_of: int | None = None          # index into ModelPlan.schedule whose cache this run reads


@dataclass
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: list
    schedule: list
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: tuple = ()
    max_position: int | None = None
    extra: dict = field(default_factory=dict)

    def validate(self) -> None:
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {run.layer}; there are {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, "
                                     f"which does not run before it")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, "
                                     f"which owns none")

    def manifest(self):
        """Every tensor the model reads, found by building the parts without weights."""
        import torch
        from ..parts.base import Runtime
        from .model import Model
        return Model(self, Runtime(torch.device("cpu"), torch.bfloat16)).tensors()
