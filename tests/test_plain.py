"""The plain implementation: checked against kishida/questwend's own CPU code (tests/golden, made
by make_golden.py from a CMake build of the reference) and against properties of its parts (no GPU)."""
import hashlib
import os

import numpy as np
import pytest

import plain_model as pm
from helpers import TINY, make_folder

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_against_the_reference(name, tmp_path):
    cfgd, seed = TINY[name]
    gold = np.load(os.path.join(GOLDEN, f"qwen3_tiny_{name}.npz"))
    folder = make_folder(tmp_path / "m", cfgd, seed, "float32")
    sha = hashlib.sha256(open(os.path.join(folder, "model.safetensors"), "rb").read()).hexdigest()
    if sha != str(gold["weights_sha256"]):
        pytest.skip("this machine draws other random weights than the one that made the golden file")
    cfg, w = pm.read_model_folder(folder)
    tokens = gold["tokens"].tolist()
    ref = gold["logits_token_by_token"].astype(np.float64)
    scale = np.abs(ref).max()
    # the reference keeps K and V in half precision and rounds the rotated Q and the probabilities to
    # half inside its products (core/runtime.cpp:498-504): with those roundings the two agree to a few
    # half-precision rounding flips, without them to the half-precision cache's own error
    plain16 = pm.forward_logits(cfg, w, tokens, round16="f16")
    plain = pm.forward_logits(cfg, w, tokens)
    assert np.abs(plain16 - ref).max() / scale < 2e-4
    assert np.abs(plain - ref).max() / scale < 1e-3
    assert (plain16.argmax(-1) == ref.argmax(-1)).all()
    # the reference's whole-prompt run gives its token-by-token run's last row
    assert np.abs(gold["logits_whole_last"] - ref[-1]).max() / scale < 1e-5


def _tiny_weights(name, tmp_path):
    cfgd, seed = TINY[name]
    return pm.read_model_folder(make_folder(tmp_path / name, cfgd, seed, "float32"))


def test_causality_and_prefix_invariance(tmp_path):
    cfg, w = _tiny_weights("B", tmp_path)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, cfg["vocab_size"], 20).tolist()
    full = pm.forward_logits(cfg, w, toks)
    assert np.allclose(pm.forward_logits(cfg, w, toks[:11]), full[:11], atol=1e-12)
    changed = toks[:15] + [(toks[15] + 1) % cfg["vocab_size"]] + toks[16:]
    other = pm.forward_logits(cfg, w, changed)
    assert np.allclose(other[:15], full[:15], atol=1e-12) and not np.allclose(other[15:], full[15:])


def test_parts():
    rng = np.random.default_rng(1)
    x = rng.normal(size=(5, 12))
    y = pm.rms_norm(x, np.ones(12), 0.0)
    assert np.allclose((y * y).mean(-1), 1.0)
    assert np.allclose(pm.rms_norm(x, np.full(12, 2.0), 1e-6), 2 * pm.rms_norm(x, np.ones(12), 1e-6))
    # rotation keeps each pair's length; position 0 is the identity; dims beyond n_rot pass through
    h = rng.normal(size=(4, 3, 16))
    ang = pm.rope_angles([0, 1, 7, 1000], 8, 10000.0)
    r = pm.apply_rope_neox(h, ang, 8)
    assert np.allclose(r[0], h[0]) and np.allclose(r[..., 8:], h[..., 8:])
    assert np.allclose(r[..., :4] ** 2 + r[..., 4:8] ** 2, h[..., :4] ** 2 + h[..., 4:8] ** 2)
    assert np.allclose(ang[3, 1], 1000 * 10000.0 ** (-2 / 8))
    # the score of rotated q and k depends on the distance only
    q, k = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    def score(pq, pk):
        return float((pm.apply_rope_neox(q, pm.rope_angles([pq], 8, 100.0), 8) *
                      pm.apply_rope_neox(k, pm.rope_angles([pk], 8, 100.0), 8)).sum())
    assert abs(score(5, 2) - score(105, 102)) < 1e-9
    # attention: first row copies v0; grouped heads read the right kv head; a window hides old keys
    T, Hq, Hkv, hd = 6, 4, 2, 8
    q, k, v = rng.normal(size=(T, Hq, hd)), rng.normal(size=(T, Hkv, hd)), rng.normal(size=(T, Hkv, hd))
    o = pm.attention_causal(q, k, v)
    assert np.allclose(o[0, 0], v[0, 0]) and np.allclose(o[0, 3], v[0, 1])
    ow = pm.attention_causal(q, k, v, window=1)
    assert np.allclose(ow[:, 1], v[:, 0]) and np.allclose(ow[:, 2], v[:, 1])
    big = q.copy(); big[5] *= 0; kk = k.copy()
    assert np.allclose(pm.attention_causal(big, kk, v)[5, 0], v[:, 0].mean(0))      # equal scores: the mean
    g = np.array([[-2.0, 0.0, 3.0]])
    assert np.allclose(pm.swiglu(g, np.ones_like(g)), g / (1 + np.exp(-g)))
    assert np.allclose(pm.round_bf16(np.array([1.0, 1.00390625, 1.005859375])), [1.0, 1.0, 1.0078125])


def test_sampler_decisions():
    lg = np.array([1.0, 3.0, 2.0, 3.0, -1.0, 0.5])
    p = pm.candidate_probabilities(lg, 1.0, top_k=3, top_p=1.0)
    assert set(np.nonzero(p)[0]) == {1, 2, 3} and abs(p.sum() - 1) < 1e-12 and p[1] == p[3]
    p = pm.candidate_probabilities(lg, 0.5, top_k=0, top_p=0.6)
    assert set(np.nonzero(p)[0]) == {1, 3}
    out = pm.penalized_logits(lg, [1, 1, 4, 9], repeat_penalty=2.0, presence=0.5, frequency=0.25)
    assert np.allclose(out, [1.0, 3.0 / 2 - 0.5 - 0.5, 2.0, 3.0, -1.0 * 2 - 0.5 - 0.25, 0.5])


def test_greedy_continue_stops(tmp_path):
    cfg, w = _tiny_weights("B", tmp_path)
    out = pm.greedy_continue(cfg, w, [3, 14, 15], 6)
    assert len(out) == 6
    assert pm.greedy_continue(cfg, w, [3, 14, 15], 6, stop_ids=(out[2],)) == out[:out.index(out[2])]
