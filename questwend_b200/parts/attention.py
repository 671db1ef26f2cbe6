"""Grouped-query attention over the paged cache, with optional per-head q/k norm, a position
encoding applied to q and k, and an optional window.  The reference's order (core/runtime.cpp:
1039-1058, 681-734): project, split heads, norm q and k (same eps), rotate, store k and v, attend
with scale 1/sqrt(head size), project back."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..kernels.limits import head_dim_refusal
from ..weights.manifest import MATRIX, NORM_WEIGHT, VECTOR, TensorSpec
from .base import KVSpec, Mixer, take_weight
from .linear import kernel_modules as linear_modules, linear, linear_onto
from .registry import register_mixer

FUSED_DECODE_MAX_BATCH = 16     # up to here a kernel less per layer pays (3-4 % of a small model's step); with more sequences
                                # every attention block repeating the work on q costs more than it saves (measured at 64).
                                # (Beyond a few rows a step's products change kernels too, so a step's arithmetic differs in
                                # its last bits between small and large batches anyway.)
DECODE_SPLIT_TOKENS = 256     # keys per run of the plain decode kernel; fixed, so results do not depend on the batch
                              # (the tensor-core kernel cuts by each sequence's own length: ops.attn_decode)


class GroupedQueryAttention(Mixer):
    """params: hidden_size, n_heads, n_kv_heads, head_dim, qk_norm (bool), norm_eps, window (0: none),
    scale (default 1/sqrt(head_dim)), names (optional overrides of the tensor names)."""

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv_heads = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("norm_eps", 0.0))
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        self.position = position
        self.rotary_dim = getattr(position, "rotary_dim", 0) if position is not None else 0
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads are not a multiple of {self.n_kv_heads} key/value heads")
        refusal = head_dim_refusal(self.head_dim)           # now, and not at the first step with the weights loaded
        if refusal:
            raise ValueError(f"grouped-query attention '{self.prefix}': parameter 'head_dim': {refusal}")
        if self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} exceeds the head size {self.head_dim}")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    def tensors(self):
        q, kv, hd, D = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.head_dim, self.hidden
        n = self.names
        out = [TensorSpec(self.prefix + n["q"], (q, D), MATRIX), TensorSpec(self.prefix + n["k"], (kv, D), MATRIX),
               TensorSpec(self.prefix + n["v"], (kv, D), MATRIX), TensorSpec(self.prefix + n["o"], (D, q), MATRIX)]
        if self.qk_norm:
            out += [TensorSpec(self.prefix + n["q_norm"], (hd,), VECTOR, NORM_WEIGHT),
                    TensorSpec(self.prefix + n["k_norm"], (hd,), VECTOR, NORM_WEIGHT)]
        return out

    def bind(self, weights):
        n, px = self.names, self.prefix
        # one fused projection: rows of q, then k, then v (a row concat, no change to the math).  The three sources are
        # taken out of ``weights`` (see ``take_weight``), so that a large model does not hold them twice until every layer
        # is bound.
        self.w_qkv = torch.cat([take_weight(weights, px + n[x]) for x in "qkv"], dim=0).contiguous()
        self.w_o = weights[px + n["o"]]
        if self.qk_norm:
            self.q_norm_w = weights[px + n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm_w = weights[px + n["k_norm"]].to(torch.float32).contiguous()

    def kernel_modules(self):
        mods = ["rope_kv", *linear_modules(self.runtime.dtype)]
        if ops.mma_attention_fits(self.runtime.dtype, self.head_dim, ops.PAGE_SIZE):
            mods.append("attention_mma")
            if ops.tc_attention_fits(self.runtime.dtype, self.head_dim, ops.PAGE_SIZE, self.n_heads // self.n_kv_heads):
                mods.append("attention_tc")
        else:
            mods.append("attention")
        return tuple(mods)

    def kv_spec(self):
        return KVSpec(self.n_kv_heads, self.head_dim, self.window)

    adds_to_residual = True

    def forward(self, x, ctx, cache, residual=None):
        qkv = linear(x, self.w_qkv)
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.prepare(ctx)
        table = ctx.page_tables[cache.group_id]
        if (ctx.single_token and ctx.n_seqs <= FUSED_DECODE_MAX_BATCH and self.rotary_dim in (0, self.head_dim)
                and ops.mma_attention_fits(cache.k_pool.dtype, self.head_dim, cache.k_pool.shape[2])):
            # one token for each of a few sequences on the tensor-core path: norm, rotation and cache write happen inside
            # the attention kernel
            att = ops.attn_decode_fused(qkv, self.q_norm_w, self.k_norm_w, cos, sin, self.eps, cache.k_pool, cache.v_pool,
                                        table, ctx.seq_len, self.scale, ctx.max_len, self.n_heads, self.n_kv_heads,
                                        self.head_dim, window=self.window, store_kv=cache.writable)
        else:
            q = ops.qk_norm_rope_store(qkv, self.q_norm_w, self.k_norm_w, cos, sin, ctx.tok_seq, ctx.tok_pos, table,
                                       cache.k_pool, cache.v_pool, self.n_heads, self.n_kv_heads, self.head_dim,
                                       self.rotary_dim, self.eps, store_kv=cache.writable)
            if ctx.single_token:
                att = ops.attn_decode(q, cache.k_pool, cache.v_pool, table, ctx.seq_len, self.scale, ctx.max_len,
                                      window=self.window, split_tokens=DECODE_SPLIT_TOKENS)
            else:
                att = ops.attn_prefill(q, cache.k_pool, cache.v_pool, table, ctx.cu_seqlens, ctx.pos0, ctx.max_new,
                                       self.scale, window=self.window)
        if residual is not None:
            return linear_onto(att, self.w_o, residual)     # None: the residual sum was made in the product's epilogue
        return linear(att, self.w_o)


register_mixer("gqa", GroupedQueryAttention)
