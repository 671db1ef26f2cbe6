"""A plain, slow implementation of the Qwen3 dense decoder, written from the
formulas of kishida/questwend (file:line below are paths inside that project).

Whole sequences, no cache, one function for each part, NumPy in float64.  It
shares no code with ``questwend_b200``: it has its own safetensors reader, its
own config reading and its own sampler.  The product is tested against this
file; this file is tested once against the compiled reference (tests/golden).

Two switches let it round where a 16-bit engine rounds, so that the engines can
be compared at their own precision:

* ``round16="f16"`` rounds the rotated Q, the cached K and V and the softmax
  probabilities to IEEE half, which is what the reference's CPU path does
  through its F16 cache (core/runtime.cpp:498-504) and ggml's F16 dot products.
* ``round16="bf16"`` rounds the weights' consumers to bfloat16 at the places
  where the bfloat16 engine does: every matrix product's input, the rotated Q,
  and the cached K and V.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# --------------------------------------------------------------------------
# rounding helpers
# --------------------------------------------------------------------------
def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round float64/float32 values to the nearest bfloat16 (ties to even)."""
    f = np.ascontiguousarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    out = np.where(np.isfinite(f), out, f)
    return out.astype(np.float64)


def round_f16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float64).astype(np.float16).astype(np.float64)


def _rounder(round16):
    if round16 is None:
        return lambda a: a
    if round16 == "bf16":
        return round_bf16
    if round16 == "f16":
        return round_f16
    raise ValueError(round16)


# --------------------------------------------------------------------------
# reading a model folder (own reader; the safetensors layout is an 8-byte
# little-endian header length, a JSON header, then raw tensor bytes)
# --------------------------------------------------------------------------
_NP_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64,
              "I32": np.int32, "U8": np.uint8}


def read_safetensors(path: str) -> dict[str, np.ndarray]:
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    base = 8 + n
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        buf = raw[base + b: base + e]
        if info["dtype"] == "BF16":
            u = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32)
        else:
            arr = np.frombuffer(buf, dtype=_NP_DTYPES[info["dtype"]])
        out[name] = arr.reshape(info["shape"]).astype(np.float64)
    return out


def read_model_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------
# the parts
# --------------------------------------------------------------------------
def embed(table: np.ndarray, ids) -> np.ndarray:
    """h0[t,:] = E[id_t,:]; a row gather without scaling (core/runtime.cpp:1001)."""
    return table[np.asarray(ids, dtype=np.int64)]


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight
    multiplies as stored (core/runtime.cpp:1018-1019; ggml-cpu/ops.cpp:3828-3850)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * weight


def linear(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """y[t,n] = sum_k W[n,k] x[t,k]; no bias anywhere (core/runtime.cpp:1039-1041)."""
    return x @ weight.T


def rope_angles(positions, rotary_dim: int, theta: float) -> np.ndarray:
    """angle[p,i] = p * theta^(-2i/n_rot), i < n_rot/2 (ggml-cuda/rope.cu:168-181,
    called with freq_scale 1 and no extrapolation, core/runtime.cpp:300-301)."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    inv_freq = theta ** (-2.0 * i / rotary_dim)
    return np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]


def apply_rope_neox(x: np.ndarray, angles: np.ndarray, rotary_dim: int) -> np.ndarray:
    """NeoX / rotate-half: pairs (i, i + n_rot/2) are rotated, dims >= n_rot pass
    through (ggml-cpu/ops.cpp:5934-5950).  x is [T, heads, head_dim]."""
    half = rotary_dim // 2
    c = np.cos(angles)[:, None, :]
    s = np.sin(angles)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:rotary_dim]
    out[..., :half] = a * c - b * s
    out[..., half:rotary_dim] = a * s + b * c
    return out


def attention_causal(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int | None = None,
                     round_probs=None) -> np.ndarray:
    """softmax(q k^T / sqrt(hd) + mask) v with grouped heads: query head h reads
    key/value head h // (Hq/Hkv); key j is visible to query t when j <= t (and
    j > t - window when a window is given) (core/runtime.cpp:690, 714-733,
    3152-3158; ggml-cpu/ops.cpp:8516,8579).  q [T,Hq,hd], k/v [T,Hkv,hd]."""
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    scale = 1.0 / np.sqrt(float(hd))
    out = np.zeros_like(q)
    j = np.arange(T)
    visible = j[None, :] <= j[:, None]
    if window is not None:
        visible &= j[None, :] > (j[:, None] - window)
    for h in range(Hq):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        if round_probs is not None:
            p = round_probs(p)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """silu(g) * u with silu(x) = x / (1 + exp(-x)) (core/runtime.cpp:1074-1076;
    ggml-cuda/unary.cuh:96-98)."""
    return gate / (1.0 + np.exp(-gate)) * up


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def _dims(cfg: dict):
    D = cfg["hidden_size"]
    Hq = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads", Hq)
    hd = cfg.get("head_dim", D // Hq)
    return D, Hq, Hkv, hd


def decoder_layer(h, w, prefix, cfg, positions, round16=None, window=None):
    """One block in the reference's order (core/runtime.cpp:1015-1081)."""
    D, Hq, Hkv, hd = _dims(cfg)
    eps = cfg["rms_norm_eps"]
    theta = cfg["rope_theta"]
    r16 = _rounder(round16)
    r_in = r16 if round16 == "bf16" else (lambda a: a)      # matrix-product inputs
    T = h.shape[0]

    x = r_in(rms_norm(h, w[prefix + "input_layernorm.weight"], eps))
    q = linear(x, w[prefix + "self_attn.q_proj.weight"]).reshape(T, Hq, hd)
    k = linear(x, w[prefix + "self_attn.k_proj.weight"]).reshape(T, Hkv, hd)
    v = linear(x, w[prefix + "self_attn.v_proj.weight"]).reshape(T, Hkv, hd)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)     # before RoPE, same eps
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)     # (core/runtime.cpp:1047-1048)
    ang = rope_angles(positions, hd, theta)
    q = r16(apply_rope_neox(q, ang, hd))
    k = r16(apply_rope_neox(k, ang, hd))
    v = r16(v)
    att = attention_causal(q, k, v, window=window,
                           round_probs=r16 if round16 == "f16" else None)
    att = r_in(att.reshape(T, Hq * hd))
    h = h + linear(att, w[prefix + "self_attn.o_proj.weight"])

    x = r_in(rms_norm(h, w[prefix + "post_attention_layernorm.weight"], eps))
    a = swiglu(linear(x, w[prefix + "mlp.gate_proj.weight"]),
               linear(x, w[prefix + "mlp.up_proj.weight"]))
    h = h + linear(r_in(a), w[prefix + "mlp.down_proj.weight"])
    return h


def forward_logits(cfg: dict, w: dict, tokens, round16=None) -> np.ndarray:
    """Logits at every position of one whole sequence, [T, V] float64
    (core/runtime.cpp:976-1100, dense branch)."""
    r_in = round_bf16 if round16 == "bf16" else (lambda a: a)
    T = len(tokens)
    positions = np.arange(T)
    h = embed(w["model.embed_tokens.weight"], tokens)
    for il in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, f"model.layers.{il}.", cfg, positions, round16=round16)
    x = r_in(rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(x, head)                      # tied head: core/runtime.cpp:1093-1094


def greedy_continue(cfg, w, prompt, n_new, round16=None, stop_ids=()):
    """Greedy decoding by re-running the whole sequence each time; the lowest id
    wins a tie (core/sampler.cpp:58-62).  A stop token ends the sequence and is
    not part of the output (cli/main.cpp:417-424)."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward_logits(cfg, w, seq, round16=round16)[-1]
        nxt = int(np.argmax(logits))
        if nxt in stop_ids:
            break
        out.append(nxt)
        seq.append(nxt)
    return out


# --------------------------------------------------------------------------
# the sampler's decisions (core/sampler.cpp:38-109), without its random stream
# --------------------------------------------------------------------------
def penalized_logits(logits, recent, repeat_penalty=1.0, presence=0.0, frequency=0.0):
    """Logits of the tokens seen in the penalty window are divided (if positive)
    or multiplied (if not) by repeat_penalty, then lowered by presence +
    frequency * count (core/sampler.cpp:43-54)."""
    out = np.array(logits, dtype=np.float64)
    counts = {}
    for t in recent:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        if t < 0 or t >= len(out):
            continue
        if repeat_penalty != 1.0:
            out[t] = out[t] / repeat_penalty if out[t] > 0 else out[t] * repeat_penalty
        out[t] -= presence + frequency * c
    return out


def candidate_probabilities(logits, temperature, top_k=0, top_p=1.0):
    """The distribution the reference draws from: top-k by logit, softmax with
    temperature, smallest descending prefix whose mass reaches top_p, then
    renormalised (core/sampler.cpp:68-99).  Returns a dense vector over the vocabulary."""
    lg = np.asarray(logits, dtype=np.float64)
    n = len(lg)
    order = np.argsort(-lg, kind="stable")
    k = min(top_k, n) if top_k > 0 else n
    order = order[:k]
    p = np.exp((lg[order] - lg[order[0]]) / temperature)
    total = p.sum()
    if top_p < 1.0:
        cum = np.cumsum(p / total)
        cut = int(np.argmax(cum >= top_p)) + 1 if np.any(cum >= top_p) else len(p)
        order, p = order[:cut], p[:cut]
    dense = np.zeros(n)
    dense[order] = p / p.sum()
    return dense
