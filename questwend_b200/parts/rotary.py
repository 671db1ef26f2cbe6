"""Rotary position encoding, NeoX form: the pairs (i, i + n_rot/2) of a head are rotated by
pos * theta^(-2i/n_rot); dims from n_rot on pass through (the reference: core/runtime.cpp:300-301,
ggml-cpu/ops.cpp:5934-5950).  The inverse frequencies are made once in float64; each step's
cos/sin table is made once and shared by every layer that uses this encoding."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import PositionEncoding
from .registry import register_position


class RotaryEncoding(PositionEncoding):
    """params: theta, rotary_dim."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary size {self.rotary_dim} must be positive and even")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-2.0 * i / self.rotary_dim)).to(runtime.device)

    def kernel_modules(self):
        return ("rope_kv",)

    def prepare(self, ctx):
        key = ("rotary", id(self))
        if key not in ctx.shared:
            ctx.shared[key] = ops.rope_table(ctx.tok_pos, self.inv_freq)
        return ctx.shared[key]


register_position("rotary_neox", RotaryEncoding)
