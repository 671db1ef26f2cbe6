"""Pre-norm residual block: h += mixer(norm1(h)); h += feed_forward(norm2(h))
(the reference: core/runtime.cpp:1015-1081; for this arrangement the second norm reads the
same tensor that the second residual sum starts from, :1066-1067).  The sums are folded into
the norms (each norm takes (h, delta), writes h + delta back and norms it) or, for parts that say
``adds_to_residual``, into the epilogue of the part's last matrix product (delta is then None) - or that product
comes back as a ``SplitSum``, sums over pieces of k that the next norm adds (``settle`` adds them for a norm that
does not say ``adds_split_sums``)."""
from __future__ import annotations

from dataclasses import replace

from .base import Block
from .linear import settle
from .registry import build_part, register_block


class PreNormBlock(Block):
    """params: mixer_norm, ffn_norm (tensor-name stems of the two norms), mixer_prefix, ffn_prefix."""

    def __init__(self, spec, runtime, layer=None, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        px = spec.prefix
        self.norm1 = build_part("norm", replace(layer.norm, prefix=px + p.get("mixer_norm", "input_layernorm") + "."), runtime)
        self.norm2 = build_part("norm", replace(layer.norm, prefix=px + p.get("ffn_norm", "post_attention_layernorm") + "."), runtime)
        self.mixer = build_part("mixer", replace(layer.mixer, prefix=px + p.get("mixer_prefix", "self_attn") + "."),
                                runtime, position=position)
        self.ffn = build_part("feed_forward", replace(layer.feed_forward, prefix=px + p.get("ffn_prefix", "mlp") + "."), runtime)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def tensors(self):
        return [t for part in self.parts() for t in part.tensors()]

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def kernel_modules(self):
        return tuple(m for part in self.parts() for m in part.kernel_modules())

    def forward(self, h, delta, ctx, cache):
        x = self.norm1.forward(h, settle(h, delta, self.norm1), write_sum=True)
        if self.mixer.adds_to_residual:
            delta = self.mixer.forward(x, ctx, cache, residual=h)
        else:
            delta = self.mixer.forward(x, ctx, cache)
        x = self.norm2.forward(h, settle(h, delta, self.norm2), write_sum=True)
        if self.ffn.adds_to_residual:
            delta = self.ffn.forward(x, ctx, residual=h)
        else:
            delta = self.ffn.forward(x, ctx)
        return h, delta


register_block("pre_norm", PreNormBlock)
