"""Dense gated feed-forward: down( silu(gate(x)) * up(x) ) (the reference: core/runtime.cpp:1074-1076)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.manifest import MATRIX, TensorSpec
from .base import FeedForward, take_weight
from .linear import kernel_modules as linear_modules, linear, linear_onto, linear_swiglu
from .registry import register_feed_forward


class GatedMLP(FeedForward):
    """params: hidden_size, intermediate_size, names (optional overrides)."""

    NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.names = {**self.NAMES, **dict(spec.params.get("names", {}))}
        self.w_gate_up = self.w_down = None
        self.interleave = 0

    def tensors(self):
        n, px = self.names, self.prefix
        return [TensorSpec(px + n["gate"], (self.inter, self.hidden), MATRIX),
                TensorSpec(px + n["up"], (self.inter, self.hidden), MATRIX),
                TensorSpec(px + n["down"], (self.hidden, self.inter), MATRIX)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        gate, up = take_weight(weights, px + n["gate"]), take_weight(weights, px + n["up"])      # only copied from
        # one fused projection.  Where the sizes allow, gate and up rows are interleaved in groups of 8 features, so that the
        # products with a fused SwiGLU epilogue find both in one thread (a reordering of rows: the same numbers).
        self.interleave = ops.GATE_UP_GROUP if self.inter % ops.GATE_UP_GROUP == 0 else 0
        if self.interleave:
            self.w_gate_up = ops.interleave_gate_up(gate, up, self.interleave)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        del gate, up
        self.w_down = weights[px + n["down"]]

    def kernel_modules(self):
        return ("elementwise", *linear_modules(self.runtime.dtype))

    adds_to_residual = True

    def forward(self, x, ctx, residual=None):
        act = linear_swiglu(x, self.w_gate_up, self.runtime.dtype, self.interleave)
        if residual is not None:
            return linear_onto(act, self.w_down, residual)  # None: the residual sum was made in the product's epilogue
        return linear(act, self.w_down)


register_feed_forward("gated_mlp", GatedMLP)
