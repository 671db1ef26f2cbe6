"""The two tiny workloads as the benchmark's description words them (needs a B200).

A: prompts of 5, 9 and 17 tokens together, then 8 greedy steps, logits at every position.
B: prompts of 1, 7, 13 and 31 tokens together, then 16 steps at temperature 0.8 under a fixed sampler seed.

Both run in 32-bit and in bfloat16 against the plain implementation.  For B the tokens the engine sampled are fed
to the plain implementation (teacher forcing), and every draw is derived again from the plain implementation's
distribution (core/sampler.cpp:68-108: softmax with temperature, a walk through the kept tokens) and the uniform
number that the sampling kernel used for (seed, sequence, step).
"""
import numpy as np
import pytest
import torch

import plain_model as pm
import questwend_b200 as qw
from helpers import BF16_TOL, FP32_TOL, TINY, make_folder
from questwend_b200.engine.engine import StepEntry
from questwend_b200.kernels import ops

pytestmark = pytest.mark.gpu


def _round(dtype):
    return None if dtype == "float32" else "bf16"


def _tol(dtype):
    return FP32_TOL if dtype == "float32" else BF16_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_workload_a_greedy_with_logits_at_every_position(dtype, tmp_path):
    cfgd, seed = TINY["A"]
    folder = make_folder(tmp_path / "a", cfgd, seed, dtype)
    cfg, w = pm.read_model_folder(folder)
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, cfgd["vocab_size"], n).tolist() for n in (5, 9, 17)]
    eng = qw.Engine.from_folder(folder, dtype=dtype, max_tokens=3 * 64)
    slots = eng.open_sequences(3)
    seqs = [list(p) for p in prompts]
    rows = [[] for _ in prompts]
    logits = eng.step([StepEntry(s, p, list(range(len(p)))) for s, p in zip(slots, prompts)]).cpu().numpy()
    off = 0
    for i, p in enumerate(prompts):
        rows[i] += list(logits[off:off + len(p)])
        off += len(p)
    for _ in range(8):
        nxt = [int(np.argmax(r[-1])) for r in rows]               # the lowest id wins a tie, as np.argmax does
        for s, t in zip(seqs, nxt):
            s.append(t)
        logits = eng.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt)]).cpu().numpy()
        for i in range(3):
            rows[i].append(logits[i])
    eng.close_sequences(slots)
    for i, p in enumerate(prompts):
        ref = pm.forward_logits(cfg, w, seqs[i], round16=_round(dtype))
        got = np.stack(rows[i]).astype(np.float64)
        err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
        assert err.max() < _tol(dtype), f"prompt of {len(p)}: position {int(np.argmax(err))} is off by {err.max():.3e}"
        # the engine's greedy tokens are the plain implementation's (with its own logits), unless two logits are closer
        # than the tolerance
        plain = pm.greedy_continue(cfg, w, p, 8, round16=_round(dtype))
        for j, (a, b) in enumerate(zip(seqs[i][len(p):], plain)):
            if a != b:
                top2 = np.sort(ref[len(p) - 1 + j])[-2:]
                assert top2[1] - top2[0] <= 2 * _tol(dtype) * np.abs(ref).max(), f"prompt of {len(p)}, new token {j}"
                break
    # the same through the generation loop
    gen = qw.generate(eng, prompts, max_new_tokens=8, ignore_eos=True)
    assert [r.tokens for r in gen] == [s[len(p):] for s, p in zip(seqs, prompts)]


def uniforms(seed: int, n_seqs: int, n_steps: int) -> np.ndarray:
    """The uniform number the sampling kernel uses for every (sequence, step) under ``seed``: it depends on nothing else."""
    dev = torch.device("cuda:0")
    dummy = torch.zeros((n_seqs, 8), dtype=torch.float32, device=dev)
    seq = torch.arange(n_seqs, dtype=torch.int32, device=dev)
    out = np.zeros((n_seqs, n_steps))
    for j in range(n_steps):
        u = torch.zeros(n_seqs, dtype=torch.float64, device=dev)
        ops.sample(dummy.clone(), 1.0, top_k=0, top_p=1.0, seed=seed, sequence_index=seq, step=j, out_u=u)
        out[:, j] = u.cpu().numpy()
    return out


@pytest.mark.parametrize("use_graph", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_workload_b_sampled_at_temperature_with_a_fixed_seed(dtype, use_graph, tmp_path):
    cfgd, seed = TINY["B"]
    folder = make_folder(tmp_path / "b", cfgd, seed, dtype)
    cfg, w = pm.read_model_folder(folder)
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, cfgd["vocab_size"], n).tolist() for n in (1, 7, 13, 31)]
    temperature, sampler_seed, n_new = 0.8, 1234, 16
    sp = qw.SamplingParams(temperature=temperature, top_k=0, top_p=1.0, seed=sampler_seed)
    eng = qw.Engine.from_folder(folder, dtype=dtype, max_tokens=4 * 64)
    res = qw.generate(eng, prompts, max_new_tokens=n_new, sampling=sp, ignore_eos=True, use_graph=use_graph)
    assert all(len(r.tokens) == n_new for r in res)
    u = uniforms(sampler_seed, len(prompts), n_new)
    exact = 0
    for i, (p, r) in enumerate(zip(prompts, res)):
        ref = pm.forward_logits(cfg, w, p + r.tokens, round16=_round(dtype))      # teacher forcing
        # logits may differ by delta = tol * max|logit|: a token's share of the mass then moves by a factor within
        # exp(+-2 delta / T), and so does every cumulative sum of the walk
        delta = _tol(dtype) * np.abs(ref).max()
        slack = np.expm1(2 * delta / temperature)
        for j, tok in enumerate(r.tokens):
            probs = pm.candidate_probabilities(ref[len(p) - 1 + j], temperature)
            cum = np.cumsum(probs)
            target = u[i, j] * cum[-1]
            lo = cum[tok - 1] if tok else 0.0
            assert lo - slack <= target <= cum[tok] + slack, (
                f"sequence {i}, new token {j}: token {tok} covers [{lo:.6f}, {cum[tok]:.6f}] of the walk, "
                f"the draw was {target:.6f} (slack {slack:.2e})")
            exact += int(np.searchsorted(cum, target, side="left")) == tok
    if dtype == "float32":
        assert exact >= len(prompts) * n_new - 1          # at 1e-4 of the logits nearly every draw is the very token
