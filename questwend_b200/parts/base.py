"""Interfaces of the parts a layer is put together from.

A model is a list of layers; a layer is a block arrangement around a mixer and a
feed-forward, with its norms and the mixer's position encoding.  Every part is
built from a ``PartSpec`` (its kind and its sizes and constants) that the
architecture's plan function derives from the configuration, layer by layer.
No part knows which model it is in: it sees its own parameters, its own
tensors (by the names its spec gives) and, while stepping, the ``StepContext``.

The reference expresses the same choices as branches inside one graph builder
(``is_recurrent(il)``, ``is_moe()``, ``gated``; core/runtime.cpp:1021-1081).

To add a part: subclass the interface below, register the class under a kind
name (``register_mixer`` and friends in ``parts.registry``), and name that kind
in a plan.  Nothing else in the package has to change.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import torch

from ..weights.manifest import TensorSpec


@dataclass(frozen=True)
class PartSpec:
    """The kind of a part (a registry key) and its parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""            # the tensors of the part are named prefix + its own names


@dataclass(frozen=True)
class KVSpec:
    """What an attention-like mixer needs from the cache: keys and values per token.
    ``window`` > 0 means only the last ``window`` keys are ever read."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Per-sequence state of fixed size (a recurrent state, a convolution tail)."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """Where and how a model computes."""
    device: torch.device
    dtype: torch.dtype          # torch.bfloat16 or torch.float32: matrices, cache and matrix-product inputs


@dataclass
class StepContext:
    """One step's batch, on the device.  T new tokens of B sequences, packed in
    sequence order.  All index tensors are int32."""
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor     # [T]
    tok_seq: torch.Tensor       # [T] batch row of each token
    tok_pos: torch.Tensor       # [T] position of each token in its own sequence
    cu_seqlens: torch.Tensor    # [B + 1] start of each sequence's tokens in the packed order
    pos0: torch.Tensor          # [B] each sequence's length before this step
    seq_len: torch.Tensor       # [B] each sequence's length after this step
    slots: torch.Tensor         # [B] cache slot of each sequence: the row of its fixed-size state (``UnitCache.state``)
    max_new: int                # most new tokens of any sequence
    max_len: int                # longest sequence after this step
    single_token: bool          # every sequence brings exactly one token
    page_tables: dict           # cache group id -> [B, width] int32 pages of each sequence
    host_slots: list | None     # the slots again, as Python ints; None in a step that may be replayed from a CUDA graph
                                # (generation's single-token steps): a part that runs there reads no value on the host
    shared: dict = field(default_factory=dict)   # per-step values shared between layers (rotation tables)


class UnitCache:
    """What one scheduled layer run sees of the cache: its own keys/values and
    state, or (``writable`` False) those of the run whose cache it reads."""

    def __init__(self, group_id=None, k_pool=None, v_pool=None, state=None, writable=True):
        self.group_id = group_id
        self.k_pool = k_pool        # [n_pages, Hkv, page_size, hd] or None
        self.v_pool = v_pool
        self.state = state          # [n_slots, *shape] or None
        self.writable = writable


def take_weight(weights, name: str) -> torch.Tensor:
    """A tensor that the caller copies into a layout of its own (a fused matrix) and does not keep as it is.  When a
    whole model is bound, ``weights`` lets go of such a tensor unless another part asks for it too, so that a large model
    is not held twice until every layer is bound; a plain dict just hands it out."""
    take = getattr(weights, "take", None)
    return take(name) if take is not None else weights[name]


class BoundWeights:
    """The tensors of a model while its parts bind them: ``weights[name]`` to keep a tensor as it is, ``take(name)`` for
    one that is only copied from.  ``uses`` counts how many parts name each tensor."""

    def __init__(self, tensors: dict, uses: Mapping[str, int]):
        self._tensors = tensors
        self._uses = dict(uses)

    def __getitem__(self, name):
        return self._tensors[name]

    def __contains__(self, name):
        return name in self._tensors

    def take(self, name):
        self._uses[name] = self._uses.get(name, 1) - 1
        return self._tensors.pop(name) if self._uses[name] <= 0 else self._tensors[name]


class Part:
    """Common to all parts: the tensors it wants and how it takes them."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.prefix = spec.prefix

    def tensors(self) -> list[TensorSpec]:
        """Every tensor of this part, with its full name and shape."""
        return []

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        """Take this part's tensors out of ``weights`` (name -> device tensor)."""

    def kernel_modules(self) -> tuple:
        """Names of the kernel modules this part launches (compiled before the first step)."""
        return ()


class Norm(Part):
    """y = norm(x + delta) over rows; x float32 [T, D]."""

    adds_split_sums = False     # True: ``delta`` may also be a SplitSum (a product left as sums over pieces of k)

    def forward(self, x, delta=None, write_sum=False, rows=None, out_dtype=None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Gives a mixer what it needs to encode positions (for a rotation: cos and sin of
    this step's tokens, made once per step and shared by all layers that use the same encoding)."""

    def prepare(self, ctx: StepContext):
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the positions of a sequence (attention here).
    x [T, D] in the engine's dtype -> float32 [T, D], to be added to the residual stream."""

    def kv_spec(self) -> KVSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    adds_to_residual = False    # True: forward(..., residual=h) adds its output onto h in place and returns None, or
                                # returns what is still to be added (a tensor, or a SplitSum that the next norm adds)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: UnitCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """Position-wise: x [T, D] in the engine's dtype -> float32 [T, D]."""

    adds_to_residual = False    # as for Mixer

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """The arrangement of norms, mixer and feed-forward around the residual stream.
    Takes and returns (h, delta): the stream and a term still to be added to it, so
    that the sum can be folded into the next norm."""

    mixer: Mixer

    def forward(self, h, delta, ctx: StepContext, cache: UnitCache):
        raise NotImplementedError
