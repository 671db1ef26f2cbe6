"""Toy parts, defined here and registered without touching the library's files: a feed-forward that routes
each token to one of a few small experts, a position encoding other than the library's own, and a norm other
than the library's own.  They show
that a layer's parts are chosen by kind, layer by layer, and that the step function, the cache and the
schedule do not care what the parts are.  The toys are written with torch operations; they are a test's
toys, not anyone's model (needs a B200)."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_model as pm
from helpers import BF16_TOL, FP32_TOL, rel_err
from questwend_b200.cache import CacheManager
from questwend_b200.config import ConfigReader, ModelConfig, register_architecture
from questwend_b200.engine.engine import Engine, StepEntry, build_step_context
from questwend_b200.engine.plan import LayerSpec, ModelPlan, Run
from questwend_b200.parts import (FeedForward, Norm, PartSpec, PositionEncoding, Runtime, build_part, register_feed_forward,
                                  register_norm, register_position)
from questwend_b200.weights import MATRIX, NORM_WEIGHT, VECTOR, TensorSpec, random_tensors

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def f64(t):
    return t.detach().to(torch.float64).cpu().numpy()


# ----------------------------------------------------------------------------- a feed-forward with routing
class TopOneExperts(FeedForward):
    """y = W2[e] relu(W1[e] x) with e = argmax(R x), the router's scores in 32-bit; the lowest index wins a tie."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.inner, self.n_experts = p["hidden_size"], p["inner_size"], p["n_experts"]

    def tensors(self):
        out = [TensorSpec(self.prefix + "router.weight", (self.n_experts, self.hidden), MATRIX)]
        for e in range(self.n_experts):
            out += [TensorSpec(f"{self.prefix}experts.{e}.w1.weight", (self.inner, self.hidden), MATRIX),
                    TensorSpec(f"{self.prefix}experts.{e}.w2.weight", (self.hidden, self.inner), MATRIX)]
        return out

    def bind(self, weights):
        self.router = weights[self.prefix + "router.weight"].float()
        self.w1 = torch.stack([weights[f"{self.prefix}experts.{e}.w1.weight"] for e in range(self.n_experts)]).float()
        self.w2 = torch.stack([weights[f"{self.prefix}experts.{e}.w2.weight"] for e in range(self.n_experts)]).float()

    def forward(self, x, ctx):
        xf = x.float()
        choice = torch.argmax(xf @ self.router.T, dim=-1)                # [T]; argmax returns the first maximum
        hidden = torch.relu(torch.einsum("tik,tk->ti", self.w1[choice], xf)).to(x.dtype).float()
        return torch.einsum("tdi,ti->td", self.w2[choice], hidden)


def plain_top_one(x, w, prefix, n_experts, rounder):
    scores = x @ w[prefix + "router.weight"].T
    choice = np.argmax(scores, axis=-1)
    out = np.zeros_like(x)
    for t, e in enumerate(choice):
        hid = rounder(np.maximum(w[f"{prefix}experts.{e}.w1.weight"] @ x[t], 0.0))
        out[t] = w[f"{prefix}experts.{e}.w2.weight"] @ hid
    return out, choice


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_feed_forward_part_alone(dtype):
    register_feed_forward("toy_top_one", TopOneExperts, replace=True)
    rt = Runtime(DEV, dtype)
    part = build_part("feed_forward", PartSpec("toy_top_one", {"hidden_size": 24, "inner_size": 40, "n_experts": 3},
                                               prefix="ff."), rt)
    w = random_tensors(part.tensors(), 5, dtype, device="cpu")
    part.bind({k: v.to(DEV) for k, v in w.items()})
    wn = {k: f64(v) for k, v in w.items()}
    x = torch.randn(50, 24, device=DEV).to(dtype)
    ref, choice = plain_top_one(f64(x), wn, "ff.", 3, pm._rounder(None if dtype == torch.float32 else "bf16"))
    assert len(set(choice.tolist())) == 3                                # every expert is used by some token
    assert rel_err(f64(part.forward(x, None)), ref) < (FP32_TOL if dtype == torch.float32 else BF16_TOL)


# ----------------------------------------------------------------------------- another position encoding
class SlowedRotary(PositionEncoding):
    """A rotation whose angle grows with pos / slowdown, on the first ``rotary_dim`` values of a head: it hands
    the mixer the same kind of table as the library's rotation, [T, rotary_dim / 2] cos and sin in 32-bit,
    made once per step and shared by the layers that use it."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.slowdown = float(spec.params["slowdown"])
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64, device=runtime.device)
        self.inv_freq = float(spec.params["theta"]) ** (-2.0 * i / self.rotary_dim)
        self.calls = 0

    def prepare(self, ctx):
        key = ("slowed", id(self))
        if key not in ctx.shared:
            self.calls += 1
            ang = (ctx.tok_pos.double() / self.slowdown)[:, None] * self.inv_freq[None, :]
            ctx.shared[key] = (torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous())
        return ctx.shared[key]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_another_position_encoding(dtype):
    register_position("toy_slowed_rotary", SlowedRotary, replace=True)
    D, Hq, Hkv, hd, rot = 48, 6, 3, 32, 16
    rt = Runtime(DEV, dtype)
    pos = build_part("position", PartSpec("toy_slowed_rotary", {"theta": 100.0, "rotary_dim": rot, "slowdown": 2.5}), rt)
    part = build_part("mixer", PartSpec("gqa", {"hidden_size": D, "n_heads": Hq, "n_kv_heads": Hkv, "head_dim": hd},
                                        prefix="a."), rt, position=pos)
    w = random_tensors(part.tensors(), 11, dtype, device="cpu")
    part.bind({k: v.to(DEV) for k, v in w.items()})
    wn = {k: f64(v) for k, v in w.items()}
    cache = CacheManager([(part.kv_spec(), None, None)], 512, 2, 256, dtype, DEV)
    unit = cache.unit_cache(0)
    T, extra = 37, 4
    x = np.random.default_rng(2).normal(size=(T + extra, D))
    rr = pm._rounder(None if dtype == torch.float32 else "bf16")
    x = rr(x)
    ang = pm.rope_angles(np.arange(T + extra) / 2.5, rot, 100.0)
    q = rr(pm.apply_rope_neox(pm.linear(x, wn["a.q_proj.weight"]).reshape(-1, Hq, hd), ang, rot))
    k = rr(pm.apply_rope_neox(pm.linear(x, wn["a.k_proj.weight"]).reshape(-1, Hkv, hd), ang, rot))
    v = rr(pm.linear(x, wn["a.v_proj.weight"]).reshape(-1, Hkv, hd))
    ref = pm.linear(rr(pm.attention_causal(q, k, v).reshape(-1, Hq * hd)), wn["a.o_proj.weight"])
    tol = (FP32_TOL if dtype == torch.float32 else BF16_TOL) * np.abs(ref).max()

    (slot,) = cache.open(1)
    def ctx_for(n):
        return build_step_context(cache, [StepEntry(slot, [0] * n, [])], 10 ** 6, DEV)[0]
    h = torch.zeros(T, D, device=DEV)
    part.forward(torch.as_tensor(x[:T]).to(dtype).to(DEV), ctx_for(T), unit, residual=h)
    cache.advance(slot, T)
    assert np.abs(f64(h) - ref[:T]).max() < tol
    for i in range(extra):
        h = torch.zeros(1, D, device=DEV)
        part.forward(torch.as_tensor(x[T + i:T + i + 1]).to(dtype).to(DEV), ctx_for(1), unit, residual=h)
        cache.advance(slot, 1)
        assert np.abs(f64(h)[0] - ref[T + i]).max() < tol
    assert pos.calls == 1 + extra


# ----------------------------------------------------------------------------- both in one toy architecture
@dataclass(frozen=True)
class ToyRoutedConfig(ModelConfig):
    hidden_size: int
    vocab_size: int
    n_experts: int
    architecture = "ToyRoutedForCausalLM"

    @classmethod
    def from_reader(cls, r: ConfigReader):
        return cls(r.integer("hidden_size"), r.integer("vocab_size"), r.integer("n_experts"))

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "n_experts": self.n_experts}


def toy_routed_plan(cfg: ToyRoutedConfig) -> ModelPlan:
    D = cfg.hidden_size
    norm = PartSpec("rms", {"dim": D, "eps": 1e-6})
    dense = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": 3 * D})
    routed = PartSpec("toy_top_one", {"hidden_size": D, "inner_size": 2 * D, "n_experts": cfg.n_experts})
    wide = PartSpec("gqa", {"hidden_size": D, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16, "qk_norm": True, "norm_eps": 1e-6})
    narrow = PartSpec("gqa", {"hidden_size": D, "n_heads": 3, "n_kv_heads": 1, "head_dim": 32, "window": 24})
    slowed = PartSpec("toy_slowed_rotary", {"theta": 1e3, "rotary_dim": 16, "slowdown": 3.0})
    rope = PartSpec("rotary_neox", {"theta": 1e4, "rotary_dim": 32})
    block = lambda i: PartSpec("pre_norm", {}, prefix=f"layers.{i}.")
    # different mixers, feed-forwards and position encodings in different layers; two cache groups (one with a window)
    layers = [LayerSpec(block(0), wide, routed, norm, slowed), LayerSpec(block(1), narrow, dense, norm, rope),
              LayerSpec(block(2), wide, routed, norm, slowed)]
    return ModelPlan(architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab_size,
                     embedding=PartSpec("token", {"vocab_size": cfg.vocab_size, "hidden_size": D, "name": "emb.weight"}),
                     layers=layers, schedule=[Run(0), Run(1), Run(2)],
                     final_norm=PartSpec("rms", {"dim": D, "eps": 1e-6}, prefix="norm."),
                     head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "hidden_size": D, "tied": False,
                                              "tied_to": "emb.weight"}))


def toy_routed_plain_logits(w, toks, n_experts):
    """The toy architecture of ``toy_routed_plan`` in NumPy, whole sequence, no cache, from the parts' formulas: what
    the assembled engine is compared with (not the engine with itself)."""
    T = len(toks)
    pos = np.arange(T)
    h = w["emb.weight"][np.asarray(toks)]
    for i in range(3):
        px = f"layers.{i}."
        wide = i != 1
        Hq, Hkv, hd = (4, 2, 16) if wide else (3, 1, 32)
        x = pm.rms_norm(h, w[px + "input_layernorm.weight"], 1e-6)
        q = pm.linear(x, w[px + "self_attn.q_proj.weight"]).reshape(T, Hq, hd)
        k = pm.linear(x, w[px + "self_attn.k_proj.weight"]).reshape(T, Hkv, hd)
        v = pm.linear(x, w[px + "self_attn.v_proj.weight"]).reshape(T, Hkv, hd)
        if wide:                                        # per-head norm, then the slowed rotation over all 16 values
            q = pm.rms_norm(q, w[px + "self_attn.q_norm.weight"], 1e-6)
            k = pm.rms_norm(k, w[px + "self_attn.k_norm.weight"], 1e-6)
            ang, rot, window = pm.rope_angles(pos / 3.0, 16, 1e3), 16, None
        else:                                           # the library's rotation over all 32 values, a window of 24 keys
            ang, rot, window = pm.rope_angles(pos, 32, 1e4), 32, 24
        q, k = pm.apply_rope_neox(q, ang, rot), pm.apply_rope_neox(k, ang, rot)
        att = pm.attention_causal(q, k, v, window=window).reshape(T, Hq * hd)
        h = h + pm.linear(att, w[px + "self_attn.o_proj.weight"])
        x = pm.rms_norm(h, w[px + "post_attention_layernorm.weight"], 1e-6)
        if wide:
            ff, _ = plain_top_one(x, w, px + "mlp.", n_experts, lambda a: a)
        else:
            ff = pm.linear(pm.swiglu(pm.linear(x, w[px + "mlp.gate_proj.weight"]), pm.linear(x, w[px + "mlp.up_proj.weight"])),
                           w[px + "mlp.down_proj.weight"])
        h = h + ff
    return pm.linear(pm.rms_norm(h, w["norm.weight"], 1e-6), w["lm_head.weight"])


def test_toy_architecture_with_routing_and_two_position_encodings(tmp_path):
    import questwend_b200 as qw
    register_feed_forward("toy_top_one", TopOneExperts, replace=True)
    register_position("toy_slowed_rotary", SlowedRotary, replace=True)
    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig, toy_routed_plan, replace=True)
    folder = qw.write_model_folder(str(tmp_path / "toy"), ToyRoutedConfig(48, 61, 3), 3, "float32")
    w = {k: v.astype(np.float64) for k, v in pm.read_safetensors(folder + "/model.safetensors").items()}
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512)
    assert eng.cache.n_groups() == 2                                     # heads 2x16 without window, 1x32 with one
    rng = np.random.default_rng(4)
    seqs = [rng.integers(0, 61, n).tolist() for n in (41, 7, 90)]
    slots = eng.open_sequences(3)
    whole = eng.step([StepEntry(s, t, list(range(len(t)))) for s, t in zip(slots, seqs)]).cpu().numpy()
    eng.close_sequences(slots)
    # the assembled toy against its NumPy model: every row of every sequence
    ref = np.concatenate([toy_routed_plain_logits(w, t, 3) for t in seqs])
    assert rel_err(whole, ref) < FP32_TOL
    # again, each alone: a prompt, then the last 6 tokens one by one, in slots that were used before
    off = 0
    for t in seqs:
        (slot,) = eng.open_sequences(1)
        cut = len(t) - 6
        rows = list(eng.step([StepEntry(slot, t[:cut], list(range(cut)))]).cpu().numpy())
        for tok in t[cut:]:
            rows.append(eng.step([StepEntry(slot, [tok], [0])]).cpu().numpy()[0])
        eng.close_sequences([slot])
        assert rel_err(np.stack(rows), whole[off:off + len(t)]) < FP32_TOL
        off += len(t)
    assert eng.cache.slots.n_free == eng.max_batch


# ----------------------------------------------------------------------------- another norm
class CenteredNorm(Norm):
    """y = c * rsqrt(mean(c^2) + eps) * w with c = v - mean(v), v = x (+ delta).  params: dim, eps; tensor: <prefix>weight.
    It does not say ``adds_split_sums``: a product that was left as sums over pieces of k is added onto the residual
    stream before this norm is called, and it never sees one."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.dim, self.eps, self.weight = int(spec.params["dim"]), float(spec.params["eps"]), None
        self.saw = []

    def tensors(self):
        return [TensorSpec(self.prefix + "weight", (self.dim,), VECTOR, NORM_WEIGHT)]

    def bind(self, weights):
        self.weight = weights[self.prefix + "weight"].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ()

    def forward(self, x, delta=None, write_sum=False, rows=None, out_dtype=None):
        self.saw.append(type(delta).__name__)
        v = x if delta is None else x + delta
        if write_sum and delta is not None:
            x.copy_(v)
        if rows is not None:
            v = v[rows.long()]
        c = v - v.mean(dim=1, keepdim=True)
        return (c * torch.rsqrt((c * c).mean(dim=1, keepdim=True) + self.eps) * self.weight).to(out_dtype or self.runtime.dtype)


@dataclass(frozen=True)
class ToyCenteredConfig(ModelConfig):
    hidden_size: int
    vocab_size: int
    eps: float
    architecture = "ToyCenteredForCausalLM"

    @classmethod
    def from_reader(cls, r: ConfigReader):
        return cls(r.integer("hidden_size"), r.integer("vocab_size"), r.number("eps"))

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "eps": self.eps}


def toy_centered_plan(cfg: ToyCenteredConfig) -> ModelPlan:
    D = cfg.hidden_size
    norm = PartSpec("toy_centered", {"dim": D, "eps": cfg.eps})
    layer = lambda i: LayerSpec(PartSpec("pre_norm", {}, prefix=f"layers.{i}."),
                                PartSpec("gqa", {"hidden_size": D, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16}),
                                PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": 72}), norm,
                                PartSpec("rotary_neox", {"theta": 1e4, "rotary_dim": 16}))
    return ModelPlan(architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab_size,
                     embedding=PartSpec("token", {"vocab_size": cfg.vocab_size, "hidden_size": D, "name": "emb.weight"}),
                     layers=[layer(0), layer(1)], schedule=[Run(0), Run(1)],
                     final_norm=PartSpec("toy_centered", {"dim": D, "eps": cfg.eps}, prefix="norm."),
                     head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "hidden_size": D, "tied": True,
                                              "tied_to": "emb.weight"}))


def toy_centered_plain_logits(w, toks, eps):
    """``toy_centered_plan`` in NumPy: whole sequence, no cache."""
    def norm(v, weight):
        c = v - v.mean(axis=-1, keepdims=True)
        return c / np.sqrt((c * c).mean(axis=-1, keepdims=True) + eps) * weight

    T = len(toks)
    h = w["emb.weight"][np.asarray(toks)]
    ang = pm.rope_angles(np.arange(T), 16, 1e4)
    for i in range(2):
        px = f"layers.{i}."
        x = norm(h, w[px + "input_layernorm.weight"])
        q = pm.apply_rope_neox(pm.linear(x, w[px + "self_attn.q_proj.weight"]).reshape(T, 4, 16), ang, 16)
        k = pm.apply_rope_neox(pm.linear(x, w[px + "self_attn.k_proj.weight"]).reshape(T, 2, 16), ang, 16)
        v = pm.linear(x, w[px + "self_attn.v_proj.weight"]).reshape(T, 2, 16)
        h = h + pm.linear(pm.attention_causal(q, k, v).reshape(T, 64), w[px + "self_attn.o_proj.weight"])
        x = norm(h, w[px + "post_attention_layernorm.weight"])
        h = h + pm.linear(pm.swiglu(pm.linear(x, w[px + "mlp.gate_proj.weight"]), pm.linear(x, w[px + "mlp.up_proj.weight"])),
                          w[px + "mlp.down_proj.weight"])
    return pm.linear(norm(h, w["norm.weight"]), w["emb.weight"])


def test_toy_architecture_with_another_norm(tmp_path, monkeypatch):
    """A norm registered from here takes the library norm's place in the blocks and before the head: the 32-bit engine
    against the NumPy model of the toy; then the bfloat16 engine with its o and down products forced into the ring
    product's split form, whose sums over pieces of k this norm cannot add: the block adds them first, the norm sees
    tensors only, and the logits are the ones without the split form, beyond rounding; generation from graphs gives the
    tokens of generation without them."""
    import questwend_b200 as qw
    from questwend_b200.kernels import ops
    register_norm("toy_centered", CenteredNorm, replace=True)
    register_architecture("ToyCenteredForCausalLM", ToyCenteredConfig, toy_centered_plan, replace=True)
    rng = np.random.default_rng(8)
    seqs = [rng.integers(0, 53, n).tolist() for n in (23, 5, 38)]
    folder, ref = {}, {}
    for dtype in ("float32", "bfloat16"):
        folder[dtype] = qw.write_model_folder(str(tmp_path / dtype), ToyCenteredConfig(40, 53, 1e-5), 5, dtype)
        w = {k: v.astype(np.float64) for k, v in pm.read_safetensors(folder[dtype] + "/model.safetensors").items()}
        ref[dtype] = [toy_centered_plain_logits(w, t, 1e-5) for t in seqs]

    def run(eng):                       # a batch of unequal prompts cut 4 tokens before their ends, then token by token
        slots = eng.open_sequences(3)
        rows = [list(r) for r in np.split(eng.step([StepEntry(s, t[:-4], list(range(len(t) - 4))) for s, t in zip(slots, seqs)])
                                          .cpu().numpy(), np.cumsum([len(t) - 4 for t in seqs])[:-1])]
        for i in range(4):
            out = eng.step([StepEntry(s, [t[len(t) - 4 + i]], [0]) for s, t in zip(slots, seqs)]).cpu().numpy()
            for r, o in zip(rows, out):
                r.append(o)
        eng.close_sequences(slots)
        return [np.stack(r) for r in rows]

    eng = Engine.from_folder(folder["float32"], dtype="float32", max_tokens=512)
    for got, want in zip(run(eng), ref["float32"]):
        assert rel_err(got, want) < FP32_TOL
    plain = run(Engine.from_folder(folder["bfloat16"], dtype="bfloat16", max_tokens=512))
    for got, want in zip(plain, ref["bfloat16"]):
        assert rel_err(got, want) < 4 * BF16_TOL                        # the NumPy model rounds no activation to 16 bits

    used = []

    def forced(N, K, n_sm, device):
        blocks = min(5, -(-N // 16) * -(-K // 256))
        counts = ops.ring_split_counts(N, K, blocks)
        if max(counts) > ops.RING_SPLIT_MAX_PLANES:
            return None
        used.append((N, K))
        return blocks, max(counts), torch.tensor(counts, dtype=torch.uint8, device=device)

    monkeypatch.setattr(ops, "_ring_split_plan", forced)
    monkeypatch.setattr(ops, "_RING_PLANS", {})
    eng = Engine.from_folder(folder["bfloat16"], dtype="bfloat16", max_tokens=512)
    split = run(eng)
    assert used, "no matrix took the split form"
    for got, want in zip(split, plain):
        assert rel_err(got, want) < BF16_TOL
    norms = [p for b in eng.model.blocks for p in (b.norm1, b.norm2)] + [eng.model.final_norm]
    assert all(isinstance(n, CenteredNorm) for n in norms)
    assert {kind for n in norms for kind in n.saw} <= {"Tensor", "NoneType"}
    prompts = [[3, 14, 15, 9, 26], [35, 8, 7], [32, 38, 46, 26, 43, 38, 32]]
    with_graphs = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=10, ignore_eos=True)]
    assert with_graphs == [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=10, ignore_eos=True, use_graph=False)]
    assert eng.cache.slots.n_free == eng.max_batch
