"""Trace replay through bin/trace_run: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths whose shorter requests end earlier, one batch after another so that
slots and pages are used again; in 32-bit and in bfloat16; all compared with the plain implementation
(needs a B200)."""
import numpy as np
import pytest

import plain_model as pm
from helpers import BF16_TOL, FP32_TOL, TINY, make_folder, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = [40, 33, 97, 130, 36]
TAIL = 32


def build_traces(tokens):
    """Steps and, for every phase and request, where its logits rows land: {(phase, r): [(step, row), ...]}."""
    steps, where = [], {}
    n = 0

    def add(entries, end=()):
        nonlocal n
        steps.append({"step": n, "entries": entries, "end": list(end)})
        n += 1
        return n - 1

    # phase "whole": each request alone, all positions wanted
    for r, t in enumerate(tokens):
        s = add([{"id": f"w{r}", "tokens": t, "want": list(range(len(t)))}], end=[f"w{r}"])
        where[("whole", r)] = [(s, i) for i in range(len(t))]
    # phase "tail": the prompt without its last 32 tokens, then those one by one
    for r, t in enumerate(tokens):
        head = len(t) - TAIL
        s = add([{"id": f"t{r}", "tokens": t[:head], "want": list(range(head))}])
        rows = [(s, i) for i in range(head)]
        for j in range(head, len(t)):
            s = add([{"id": f"t{r}", "tokens": [t[j]], "want": [0]}], end=[f"t{r}"] if j == len(t) - 1 else [])
            rows.append((s, 0))
        where[("tail", r)] = rows
    # phase "batch": requests start together with unequal prompts, go on one token each; shorter ones end earlier;
    # the second batch starts when the first is over and gets its slots and pages
    for members, heads in (([0, 1, 2], [7, 30, 64]), ([3, 4, 0], [100, 1, 12])):
        rows = {r: [] for r in members}
        entries, row = [], 0
        for r, h in zip(members, heads):
            entries.append({"id": f"b{r}", "tokens": tokens[r][:h], "want": list(range(h))})
        pos = dict(zip(members, heads))
        ends = [f"b{r}" for r in members if pos[r] == len(tokens[r])]
        s = add(entries, end=ends)
        for r, h in zip(members, heads):
            rows[r] += [(s, row + i) for i in range(h)]
            row += h
        live = [r for r in members if pos[r] < len(tokens[r])]
        while live:
            entries = [{"id": f"b{r}", "tokens": [tokens[r][pos[r]]], "want": [0]} for r in live]
            for r in live:
                pos[r] += 1
            ends = [f"b{r}" for r in live if pos[r] == len(tokens[r])]
            s = add(entries, end=ends)
            for i, r in enumerate(live):
                rows[r].append((s, i))
            live = [r for r in live if pos[r] < len(tokens[r])]
        for r in members:
            where[(f"batch{members[0]}", r)] = rows[r]
    return steps, where


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_agrees_with_the_plain_implementation(name, dtype, tmp_path):
    cfgd, seed = TINY[name]
    folder = make_folder(tmp_path / "model", cfgd, seed, dtype)
    cfg, w = pm.read_model_folder(folder)
    rng = np.random.default_rng(seed + 10)
    tokens = [rng.integers(0, cfgd["vocab_size"], n).tolist() for n in LENGTHS]
    steps, where = build_traces(tokens)
    # the most that live requests hold, each rounded up to 64: the second batch (130, 36, 40 tokens)
    out = run_trace(folder, dtype, steps, max_tokens=192 + 64 + 64, out_dir=str(tmp_path / "out"))
    tol = FP32_TOL if dtype == "float32" else BF16_TOL
    refs = [pm.forward_logits(cfg, w, t, round16=None if dtype == "float32" else "bf16") for t in tokens]
    got_whole = {}
    for (phase, r), rows in where.items():
        got = np.stack([out[s][i] for s, i in rows]).astype(np.float64)
        ref = refs[r]
        scale = np.abs(ref).max()
        err = np.abs(got - ref).max(axis=1) / scale
        first_bad = int(np.argmax(err > tol)) if (err > tol).any() else -1
        assert first_bad < 0, (f"{phase}, request {r}: position {first_bad} of {len(ref)} is off by "
                               f"{err[first_bad]:.3e} (tolerance {tol:.1e})")
        # the engine's greedy token is the plain implementation's, unless the two best logits are closer
        # than the tolerance
        top2 = np.sort(ref, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2 * tol * scale
        assert (got.argmax(1) == ref.argmax(1))[clear].all()
        if phase == "whole":
            got_whole[r] = got
        else:                                                 # the ways of cutting agree with each other
            assert np.abs(got - got_whole[r]).max() / scale < tol
