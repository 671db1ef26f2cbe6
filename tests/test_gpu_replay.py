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


# ---------------------------------------------------------------------------------------------------------------------
# Many live sequences.  A decode step's kernels change with its number of rows (up to 8, 9 to 16, 17 and more: other
# forms of the few-rows product, library products, the separate q/k-norm + rotation kernel), so the batches here start
# with 64 and 24 requests and shrink through 17, 16, 9, 8 and 1 as requests end.  The reference's own check of this kind
# feeds one prompt whole and token by token (cli/main.cpp:313-337).
# ---------------------------------------------------------------------------------------------------------------------
# how many requests decode for how many steps; the live count after the prompts' step is then, step by step,
# 64 64 44 17 17 16 16 9 9 8 8 4 4 1 1 1  and  24 17 16 9 8 1 1
DECODE_STEPS_1 = [2] * 20 + [3] * 27 + [5] + [7] * 7 + [9] + [11] * 4 + [13] * 3 + [16]
DECODE_STEPS_2 = [1] * 7 + [2] + [3] * 7 + [4] + [5] * 7 + [7]
LIVE_COUNTS_1 = [64, 64, 44, 17, 17, 16, 16, 9, 9, 8, 8, 4, 4, 1, 1, 1]
LIVE_COUNTS_2 = [24, 17, 16, 9, 8, 1, 1]


def many_requests(rng, vocab):
    """[(batch, prompt length, tokens)]: unequal prompts (some of one token, some across a page's edge), then as many
    single tokens as the request decodes; which request ends when is shuffled, so that the ended ones lie anywhere in
    the batch."""
    out = []
    for batch, decode_steps in enumerate((DECODE_STEPS_1, DECODE_STEPS_2)):
        steps = list(decode_steps)
        rng.shuffle(steps)
        heads = rng.integers(1, 25, len(steps)).tolist()
        heads[0], heads[1], heads[2], heads[3] = 1, 64, 63, 130
        for h, d in zip(heads, steps):
            out.append((batch, h, rng.integers(0, vocab, h + d).tolist()))
    return out


def build_many_traces(requests):
    steps, where, live_counts = [], {}, {0: [], 1: []}
    peak = 0
    for r, (_, _, t) in enumerate(requests):                       # each request alone and whole
        steps.append({"step": len(steps), "entries": [{"id": f"w{r}", "tokens": t, "want": list(range(len(t)))}],
                      "end": [f"w{r}"]})
        where[("whole", r)] = [(len(steps) - 1, i) for i in range(len(t))]
    for batch in (0, 1):                                           # the second batch gets the first one's slots and pages
        members = [r for r, q in enumerate(requests) if q[0] == batch]
        peak = max(peak, sum(-(-len(requests[r][2]) // 64) * 64 for r in members))
        pos = {r: requests[r][1] for r in members}
        rows = {r: [] for r in members}
        s, row = len(steps), 0
        for r in members:
            rows[r] += [(s, row + i) for i in range(pos[r])]
            row += pos[r]
        steps.append({"step": s, "entries": [{"id": f"m{r}", "tokens": requests[r][2][:pos[r]],
                                              "want": list(range(pos[r]))} for r in members], "end": []})
        live = list(members)
        while live:
            s = len(steps)
            live_counts[batch].append(len(live))
            entries = []
            for i, r in enumerate(live):
                entries.append({"id": f"m{r}", "tokens": [requests[r][2][pos[r]]], "want": [0]})
                rows[r].append((s, i))
                pos[r] += 1
            ended = [r for r in live if pos[r] == len(requests[r][2])]
            steps.append({"step": s, "entries": entries, "end": [f"m{r}" for r in ended]})
            live = [r for r in live if r not in ended]
        for r in members:
            where[("batch", r)] = rows[r]
    return steps, where, live_counts, peak


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_many_live_sequences(name, dtype, tmp_path):
    cfgd, seed = TINY[name]
    folder = make_folder(tmp_path / "model", cfgd, seed, dtype)
    cfg, w = pm.read_model_folder(folder)
    requests = many_requests(np.random.default_rng(seed + 40), cfgd["vocab_size"])
    steps, where, live_counts, peak = build_many_traces(requests)
    assert live_counts[0] == LIVE_COUNTS_1 and live_counts[1] == LIVE_COUNTS_2
    out = run_trace(folder, dtype, steps, max_tokens=peak, out_dir=str(tmp_path / "out"))
    tol = FP32_TOL if dtype == "float32" else BF16_TOL
    whole = {}
    for (phase, r), rows in sorted(where.items(), key=lambda kv: kv[0][0] != "whole"):
        ref = pm.forward_logits(cfg, w, requests[r][2], round16=None if dtype == "float32" else "bf16")
        got = np.stack([out[s][i] for s, i in rows]).astype(np.float64)
        scale = np.abs(ref).max()
        err = np.abs(got - ref).max(axis=1) / scale
        bad = int(np.argmax(err > tol)) if (err > tol).any() else -1
        assert bad < 0, (f"{phase}, request {r} (prompt of {requests[r][1]}): position {bad} of {len(ref)} is off by "
                         f"{err[bad]:.3e} (tolerance {tol:.1e}); step {rows[bad][0]}, row {rows[bad][1]}")
        if phase == "whole":
            whole[r] = got
        else:
            assert np.abs(got - whole[r]).max() / scale < tol, f"request {r}: in the batch it differs from alone"
