"""Each part of a layer alone, and a toy architecture with a mixer that keeps state of its own,
registered from here without touching the library's files (needs a B200)."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_model as pm
from helpers import BF16_TOL, FP32_TOL, rel_err
from questwend_b200.cache import CacheManager
from questwend_b200.kernels import ops
from questwend_b200.config import ConfigReader, ModelConfig, register_architecture
from questwend_b200.engine.engine import Engine, StepEntry, build_step_context
from questwend_b200.engine.plan import LayerSpec, ModelPlan, Run
from questwend_b200.parts import (Mixer, PartSpec, Runtime, StateSpec, build_part, register_mixer)
from questwend_b200.weights import MATRIX, TensorSpec, random_tensors

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def f64(t):
    return t.detach().to(torch.float64).cpu().numpy()


def tol(dtype):
    return FP32_TOL if dtype == torch.float32 else BF16_TOL


def r16(dtype):
    return None if dtype == torch.float32 else "bf16"


def make_part(family, spec, dtype, seed=0, **extra):
    rt = Runtime(DEV, dtype)
    part = build_part(family, spec, rt, **extra)
    w = random_tensors(part.tensors(), seed, dtype, device="cpu")
    part.bind({k: v.to(DEV) for k, v in w.items()})
    return part, {k: f64(v) for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    part, w = make_part("norm", PartSpec("rms", {"dim": 72, "eps": 1e-4}, prefix="n."), dtype)
    x = torch.randn(5, 72, device=DEV) * 2
    assert rel_err(f64(part.forward(x)), pm.rms_norm(f64(x), w["n.weight"], 1e-4)) < tol(dtype)
    assert part.forward(x).dtype == dtype and part.forward(x, out_dtype=torch.float32).dtype == torch.float32


def step_context(cache, slots, token_lists):
    return build_step_context(cache, [StepEntry(s, t, []) for s, t in zip(slots, token_lists)], 10 ** 6, DEV)[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 20])
def test_attention_part_prompt_then_tokens(dtype, window):
    D, Hq, Hkv, hd = 80, 5, 1, 48
    rt = Runtime(DEV, dtype)
    pos = build_part("position", PartSpec("rotary_neox", {"theta": 5e4, "rotary_dim": 32}), rt)
    spec = PartSpec("gqa", {"hidden_size": D, "n_heads": Hq, "n_kv_heads": Hkv, "head_dim": hd, "qk_norm": True,
                            "norm_eps": 1e-5, "window": window}, prefix="a.")
    part, w = make_part("mixer", spec, dtype, seed=3, position=pos)
    cache = CacheManager([(part.kv_spec(), None, None)], 1024, 4, 512, dtype, DEV)
    unit = cache.unit_cache(0)
    lens, extra = [70, 9, 33], 5
    rng = np.random.default_rng(1)
    xs = [rng.normal(size=(n + extra, D)) for n in lens]
    if dtype == torch.bfloat16:
        xs = [pm.round_bf16(x) for x in xs]

    def plain(x):
        T = x.shape[0]
        q = pm.rms_norm(pm.linear(x, w["a.q_proj.weight"]).reshape(T, Hq, hd), w["a.q_norm.weight"], 1e-5)
        k = pm.rms_norm(pm.linear(x, w["a.k_proj.weight"]).reshape(T, Hkv, hd), w["a.k_norm.weight"], 1e-5)
        v = pm.linear(x, w["a.v_proj.weight"]).reshape(T, Hkv, hd)
        ang = pm.rope_angles(np.arange(T), 32, 5e4)
        rr = pm._rounder(r16(dtype))
        q, k, v = rr(pm.apply_rope_neox(q, ang, 32)), rr(pm.apply_rope_neox(k, ang, 32)), rr(v)
        att = rr(pm.attention_causal(q, k, v, window=window or None).reshape(T, Hq * hd))
        return pm.linear(att, w["a.o_proj.weight"])

    refs = [plain(x) for x in xs]
    slots = cache.open(3)
    ctx = step_context(cache, slots, [[0] * n for n in lens])
    x_dev = torch.cat([torch.as_tensor(x[:n]) for x, n in zip(xs, lens)]).to(dtype).to(DEV)
    out = f64(part.forward(x_dev, ctx, unit))
    for s, n in zip(slots, lens):
        cache.advance(s, n)
    off = 0
    scale = max(np.abs(r).max() for r in refs)
    for x, n, ref in zip(xs, lens, refs):
        assert np.abs(out[off:off + n] - ref[:n]).max() / scale < tol(dtype)
        off += n
    for i in range(extra):                                  # then one token each, from the cache
        ctx = step_context(cache, slots, [[0]] * 3)
        x_dev = torch.stack([torch.as_tensor(x[n + i]) for x, n in zip(xs, lens)]).to(dtype).to(DEV)
        out = f64(part.forward(x_dev, ctx, unit))
        for b, (n, ref) in enumerate(zip(lens, refs)):
            assert np.abs(out[b] - ref[n + i]).max() / scale < tol(dtype)
        for s in slots:
            cache.advance(s, 1)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    spec = PartSpec("gated_mlp", {"hidden_size": 56, "intermediate_size": 100}, prefix="f.")
    part, w = make_part("feed_forward", spec, dtype, seed=2)
    for T in (3, 40):                                       # few rows: own kernel; many: the library product
        x = torch.randn(T, 56, device=DEV).to(dtype)
        a = pm.swiglu(pm.linear(f64(x), w["f.gate_proj.weight"]), pm.linear(f64(x), w["f.up_proj.weight"]))
        a = pm._rounder(r16(dtype))(a)
        assert rel_err(f64(part.forward(x, None)), pm.linear(a, w["f.down_proj.weight"])) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    emb, w = make_part("embedding", PartSpec("token", {"vocab_size": 50, "hidden_size": 24}, prefix="model."), dtype)
    ids = torch.tensor([3, 49, 0], dtype=torch.int32, device=DEV)
    assert np.array_equal(f64(emb.forward(ids)), w["model.embed_tokens.weight"][[3, 49, 0]])
    rt = Runtime(DEV, dtype)
    for tied in (True, False, None):
        head = build_part("head", PartSpec("linear", {"vocab_size": 50, "hidden_size": 24, "tied": tied,
                                                      "tied_to": "model.embed_tokens.weight"}), rt)
        own = torch.randn(50, 24).to(dtype)
        head.bind({"model.embed_tokens.weight": emb.table, "lm_head.weight": own.to(DEV)})
        x = torch.randn(2, 24, device=DEV).to(dtype)
        want = w["model.embed_tokens.weight"] if tied else f64(own)
        assert rel_err(f64(head.forward(x)), f64(x) @ want.T) < tol(dtype)
    head.bind({"model.embed_tokens.weight": emb.table})     # undecided and no head stored: tied
    assert head.weight is emb.table


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    cfg = {"hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
           "rms_norm_eps": 1e-6, "rope_theta": 1e4}
    layer = LayerSpec(block=PartSpec("pre_norm", {}, prefix="model.layers.0."),
                      mixer=PartSpec("gqa", {"hidden_size": 64, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16,
                                             "qk_norm": True, "norm_eps": 1e-6}),
                      feed_forward=PartSpec("gated_mlp", {"hidden_size": 64, "intermediate_size": 88}),
                      norm=PartSpec("rms", {"dim": 64, "eps": 1e-6}),
                      position=PartSpec("rotary_neox", {"theta": 1e4, "rotary_dim": 16}))
    rt = Runtime(DEV, dtype)
    pos = build_part("position", layer.position, rt)
    block, w = make_part("block", layer.block, dtype, seed=4, layer=layer, position=pos)
    cache = CacheManager([(block.mixer.kv_spec(), None, None)], 256, 2, 256, dtype, DEV)
    (slot,) = cache.open(1)
    T = 19
    h = np.random.default_rng(0).normal(size=(T, 64)).astype(np.float32)
    ref = pm.decoder_layer(h.astype(np.float64), w, "model.layers.0.", cfg, np.arange(T), round16=r16(dtype))
    ctx = step_context(cache, [slot], [[0] * T])
    h_dev, delta = block.forward(torch.from_numpy(h).to(DEV), None, ctx, cache.unit_cache(0))
    assert h_dev.dtype == torch.float32 and (delta is None or delta.dtype == torch.float32)   # a 32-bit residual stream
    assert rel_err(f64(h_dev) + (0 if delta is None else f64(delta)), ref) < tol(dtype)


def test_few_row_products_by_either_kernel(monkeypatch):
    """``linear`` with few rows: the ring-fed kernel (the default) and the kernel before it give the product's numbers, and
    from 9 rows on a large matrix goes to the library."""
    from questwend_b200.parts import linear as L
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(2560, 4096, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    for kernel in ("ring", "stream"):
        monkeypatch.setattr(L, "FEW_ROWS_KERNEL", kernel)
        for rows in (3, 8, 12):
            x = torch.randn(rows, 4096, generator=g).to(torch.bfloat16).to(DEV)
            ref = f64(x) @ f64(w).T
            before = ops.LAUNCHES[0]
            out = L.linear(x, w)
            assert ops.LAUNCHES[0] == before + 1                           # an own kernel ran, not the library
            assert rel_err(f64(out), ref) < FP32_TOL * 4                      # 32-bit sums of exact products
            base = torch.randn(rows, 2560, generator=g).to(DEV)
            added = L.linear(x, w, add_to=base.clone())
            assert rel_err(f64(added), f64(base) + ref) < FP32_TOL * 4
        gu = L.linear_swiglu(x, w, torch.bfloat16, interleave=8)             # 1280 features, gate and up interleaved in eights
        y = ref.reshape(rows, 160, 2, 8)
        assert rel_err(f64(gu), pm.swiglu(y[:, :, 0], y[:, :, 1]).reshape(rows, 1280)) < BF16_TOL
    ops.gemm_tc_check(DEV)
    monkeypatch.setattr(L, "STREAM_WIDE_MAX_WEIGHT", 1 << 20)                  # now 10 M weights count as large
    before = ops.LAUNCHES[0]
    assert rel_err(f64(L.linear(x, w)), ref) < FP32_TOL * 4 and ops.LAUNCHES[0] == before     # 12 rows: the library


# ----------------------------------------------------------------------------- a toy architecture, defined here
class RunningMeanMixer(Mixer):
    """y_t = mean(x_0..x_t) W.  Keeps, per sequence, the running sum and the count: fixed-size state, no keys or values.
    The state rows are found with ``ctx.slots`` on the device and nothing is read on the host, so a step can be replayed
    from a CUDA graph for whichever sequences are bound to it.  Written with torch operations; it is a test's toy, not a
    model."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        self.hidden = spec.params["hidden_size"]

    def tensors(self):
        return [TensorSpec(self.prefix + "w.weight", (self.hidden, self.hidden), MATRIX)]

    def bind(self, weights):
        self.w = weights[self.prefix + "w.weight"]

    def state_spec(self):
        return StateSpec((self.hidden + 1,), torch.float32)

    def forward(self, x, ctx, cache):
        seq = ctx.tok_seq.long()                                  # [T] batch row of each token
        slot = ctx.slots.long()                                   # [B] state row of each sequence
        state = cache.state.index_select(0, slot).double()        # [B, D + 1]
        running = torch.cumsum(x.double(), 0)                     # over the packed tokens; each sequence subtracts what
        first = ctx.cu_seqlens[:-1].long()                        # had run up before its own first token
        before = running.index_select(0, (first - 1).clamp(min=0)) * (first > 0)[:, None]
        sums = state[:, :-1].index_select(0, seq) + running - before.index_select(0, seq)
        counts = state[:, -1].index_select(0, seq) + (ctx.tok_pos - ctx.pos0.index_select(0, seq) + 1)
        if cache.writable:
            last = ctx.cu_seqlens[1:].long() - 1
            new = torch.cat([sums.index_select(0, last), counts.index_select(0, last)[:, None]], dim=1)
            cache.state.index_copy_(0, slot, new.float())
        return (sums / counts[:, None]).to(x.dtype).float() @ self.w.float().T


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    hidden_size: int
    vocab_size: int
    architecture = "ToyStateForCausalLM"

    @classmethod
    def from_reader(cls, r: ConfigReader):
        return cls(r.integer("hidden_size"), r.integer("vocab_size"))

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size}


def toy_plan(cfg: ToyConfig) -> ModelPlan:
    D = cfg.hidden_size
    norm = PartSpec("rms", {"dim": D, "eps": 1e-5})
    ffn = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": 2 * D})
    attn = PartSpec("gqa", {"hidden_size": D, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "qk_norm": False})
    toy = PartSpec("toy_running_mean", {"hidden_size": D})
    rope = PartSpec("rotary_neox", {"theta": 1e4, "rotary_dim": 16})
    block = lambda i: PartSpec("pre_norm", {"mixer_norm": "n1", "ffn_norm": "n2", "mixer_prefix": "mix", "ffn_prefix": "ff"},
                               prefix=f"layers.{i}.")
    layers = [LayerSpec(block(0), toy, ffn, norm), LayerSpec(block(1), attn, ffn, norm, rope),
              LayerSpec(block(2), toy, ffn, norm)]
    # layer 1 runs twice; its second run reads the first run's keys and values
    schedule = [Run(0), Run(1), Run(2), Run(1, cache_of=1), Run(0)]
    return ModelPlan(architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab_size,
                     embedding=PartSpec("token", {"vocab_size": cfg.vocab_size, "hidden_size": D, "name": "emb.weight"}),
                     layers=layers, schedule=schedule, final_norm=PartSpec("rms", {"dim": D, "eps": 1e-5}, prefix="norm."),
                     head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "hidden_size": D, "tied": True,
                                              "tied_to": "emb.weight"}))


def toy_plain_logits(w, tokens):
    """The toy architecture once more in NumPy float64, whole sequences, no cache and no state: what the engine's
    schedule, cache and state rows have to reproduce."""
    T = len(tokens)
    eps = 1e-5

    def feed_forward(h, px):
        x = pm.rms_norm(h, w[px + "n2.weight"], eps)
        a = pm.swiglu(pm.linear(x, w[px + "ff.gate_proj.weight"]), pm.linear(x, w[px + "ff.up_proj.weight"]))
        return h + pm.linear(a, w[px + "ff.down_proj.weight"])

    def running_mean(h, px):
        x = pm.rms_norm(h, w[px + "n1.weight"], eps)
        mean = np.cumsum(x, 0) / np.arange(1, T + 1)[:, None]
        return feed_forward(h + pm.linear(mean, w[px + "mix.w.weight"]), px)

    def attention(h, px, kv=None):
        x = pm.rms_norm(h, w[px + "n1.weight"], eps)
        ang = pm.rope_angles(np.arange(T), 16, 1e4)
        q = pm.apply_rope_neox(pm.linear(x, w[px + "mix.q_proj.weight"]).reshape(T, 2, 16), ang, 16)
        if kv is None:
            k = pm.apply_rope_neox(pm.linear(x, w[px + "mix.k_proj.weight"]).reshape(T, 1, 16), ang, 16)
            kv = (k, pm.linear(x, w[px + "mix.v_proj.weight"]).reshape(T, 1, 16))
        att = pm.attention_causal(q, kv[0], kv[1]).reshape(T, 32)
        return feed_forward(h + pm.linear(att, w[px + "mix.o_proj.weight"]), px), kv

    h = w["emb.weight"][np.asarray(tokens)]
    h = running_mean(h, "layers.0.")
    h, kv = attention(h, "layers.1.")
    h = running_mean(h, "layers.2.")
    h, _ = attention(h, "layers.1.", kv)              # the same layer again, with the first run's keys and values
    h = running_mean(h, "layers.0.")                  # and the first layer again, with a state of its own
    return pm.linear(pm.rms_norm(h, w["norm.weight"], eps), w["emb.weight"])


@pytest.fixture(scope="module")
def toy_model(tmp_path_factory):
    import questwend_b200 as qw
    register_mixer("toy_running_mean", RunningMeanMixer, replace=True)
    register_architecture("ToyStateForCausalLM", ToyConfig, toy_plan, replace=True)
    folder = str(tmp_path_factory.mktemp("toy_state"))
    qw.write_model_folder(folder, ToyConfig(32, 40), seed=7, dtype="float32")
    return folder, pm.read_safetensors(folder + "/model.safetensors")


def test_toy_mixer_with_state_of_its_own(toy_model):
    folder, w = toy_model
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512)
    units = eng.model.cache_units()
    assert [u[0] is not None for u in units] == [False, True, False, True, False]
    assert [u[1] is not None for u in units] == [True, False, True, False, True]
    assert eng.cache.n_groups() == 1 and not eng.unit_caches[3].writable
    assert eng.unit_caches[0].state.data_ptr() != eng.unit_caches[4].state.data_ptr()   # a layer run twice: two states
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 40, n).tolist() for n in (23, 5, 70)]
    refs = [toy_plain_logits(w, t) for t in seqs]
    slots = eng.open_sequences(3)
    whole = eng.step([StepEntry(s, t, list(range(len(t)))) for s, t in zip(slots, seqs)]).cpu().numpy()
    eng.close_sequences(slots)
    off = 0
    for t, ref in zip(seqs, refs):
        assert rel_err(whole[off:off + len(t)], ref) < FP32_TOL
        off += len(t)
    # the same sequences: a prompt of a few tokens, then token by token, in slots that were used before
    slots = eng.open_sequences(3)
    rows = {i: [] for i in range(3)}
    cuts = [4, 1, 66]
    first = eng.step([StepEntry(s, t[:c], list(range(c))) for s, t, c in zip(slots, seqs, cuts)]).cpu().numpy()
    off = 0
    for i, c in enumerate(cuts):
        rows[i] += list(first[off:off + c]); off += c
    live = [0, 1, 2]
    pos = list(cuts)
    while live:
        out = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            rows[i].append(out[r]); pos[i] += 1
        done = [i for i in live if pos[i] == len(seqs[i])]
        eng.close_sequences([slots[i] for i in done])
        live = [i for i in live if i not in done]
    for i, ref in enumerate(refs):
        assert rel_err(np.stack(rows[i]), ref) < FP32_TOL
    assert eng.cache.slots.n_free == eng.max_batch


@pytest.mark.parametrize("use_graph", [True, False])
def test_toy_state_through_the_generation_loop(toy_model, use_graph):
    """Generation's decode steps (replayed from CUDA graphs, or plain) on the model whose mixer keeps state: two batches one
    after the other, in slots that are not 0..B-1 (another sequence holds slot 0 meanwhile) and that are used again, one
    sequence ending early at a stop token.  Every token is checked against the NumPy model fed the same tokens."""
    import questwend_b200 as qw
    folder, w = toy_model
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_batch=3)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 40, n).tolist() for n in (9, 2, 30, 1, 14)]
    (held,) = eng.open_sequences(1)                          # generation gets slots 1 and 2
    assert held == 0
    eng.step([StepEntry(held, [1, 2, 3], [])])
    n_new = 14
    free = qw.generate(eng, prompts, max_new_tokens=n_new, ignore_eos=True, use_graph=use_graph)
    stop = free[2].tokens[5]                                 # ends the third sequence (at least) early
    stats = qw.GenerationStats()
    res = qw.generate(eng, prompts, max_new_tokens=n_new, stop_ids=[stop], use_graph=use_graph, stats=stats)
    assert stats.batches == 3 and res[2].finish_reason == "stop" and len(res[2].tokens) <= 5
    for run in (free, res):
        for p, r in zip(prompts, run):
            ref = toy_plain_logits(w, p + r.tokens)
            scale = np.abs(ref).max()
            for j, tok in enumerate(r.tokens):
                row = ref[len(p) - 1 + j]
                assert row.max() - row[tok] <= 2 * FP32_TOL * scale, (
                    f"prompt of {len(p)}, new token {j}: the engine chose {tok}, the NumPy model {int(row.argmax())}")
            if r.finish_reason == "stop":
                assert int(ref[len(p) - 1 + len(r.tokens)].argmax()) == stop
    eng.close_sequences([held])
    assert eng.cache.slots.n_free == eng.max_batch
