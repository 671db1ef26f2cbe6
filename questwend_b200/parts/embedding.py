"""Token embedding (a row gather, no scaling; core/runtime.cpp:1001) and the output head
(logits = x W^T with the embedding table as W when the head is tied; core/runtime.cpp:1093-1096)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.manifest import MATRIX, TensorSpec
from .base import Part
from .linear import kernel_modules as linear_modules, linear
from .registry import register_embedding, register_head


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.name = self.prefix + spec.params.get("name", "embed_tokens.weight")
        self.table = None

    def tensors(self):
        return [TensorSpec(self.name, (self.vocab, self.hidden), MATRIX)]

    def bind(self, weights):
        self.table = weights[self.name]

    def kernel_modules(self):
        return ("elementwise",)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embed_gather(token_ids, self.table)


class OutputHead(Part):
    """params: vocab_size, hidden_size, tied (True, False, or None: tied iff the head's tensor is absent),
    name, tied_to (name of the embedding table)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = spec.params.get("tied")
        self.name = self.prefix + spec.params.get("name", "lm_head.weight")
        self.tied_to = spec.params["tied_to"]
        self.weight = None

    def tensors(self):
        # tied: a stored copy may be there and is not used; undecided: the tensor's presence decides
        return [TensorSpec(self.name, (self.vocab, self.hidden), MATRIX,
                           optional=self.tied is None, ignored=self.tied is True)]

    def bind(self, weights):
        if self.tied is True or (self.tied is None and self.name not in weights):
            self.weight = weights[self.tied_to]
        else:
            self.weight = weights[self.name]

    def kernel_modules(self):
        return linear_modules(self.runtime.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight)


register_embedding("token", TokenEmbedding)
register_head("linear", OutputHead)
