"""RMS norm: y = v * rsqrt(mean(v^2) + eps) * w, v = x (+ delta), sums in 32-bit
(the reference: core/runtime.cpp:1018-1019, 1066, 1090-1091)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.manifest import NORM_WEIGHT, VECTOR, TensorSpec
from .base import Norm
from .registry import register_norm


class RMSNorm(Norm):
    """params: dim, eps; tensor: <prefix>weight [dim]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.dim = int(spec.params["dim"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensors(self):
        return [TensorSpec(self.prefix + "weight", (self.dim,), VECTOR, NORM_WEIGHT)]

    def bind(self, weights):
        self.weight = weights[self.prefix + "weight"].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ("elementwise",)

    adds_split_sums = True      # ``delta`` may be a SplitSum: the kernel adds its planes

    def forward(self, x, delta=None, write_sum=False, rows=None, out_dtype=None):
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype or self.runtime.dtype, delta=delta,
                           write_sum=write_sum, rows=rows)


register_norm("rms", RMSNorm)
