"""The generation loop's decisions, followed with a scripted engine (no GPU)."""
import pytest
import torch

from questwend_b200.cache import CacheManager
from questwend_b200.engine.generate import (FINISH_CONTEXT, FINISH_LENGTH, FINISH_STOP, GenerationStats, generate,
                                            plan_batches)
from questwend_b200.kernels.ops import PAGE_SIZE
from questwend_b200.parts.base import KVSpec
from questwend_b200.sampling import SamplingParams

V = 50


class ScriptedEngine:
    """Stands for the engine: the 'model' answers token t at position p of a sequence with the
    token (sum of the sequence so far + p) mod V; the cache is the real bookkeeping, on the CPU."""

    def __init__(self, max_tokens=16 * PAGE_SIZE, max_batch=3, max_seq_len=4 * PAGE_SIZE):
        self.cache = CacheManager([(KVSpec(1, 16), None, None)], max_tokens, max_batch, max_seq_len,
                                  torch.float32, "cpu")
        self.max_batch = max_batch
        self.device = "cpu"
        self.plan = type("P", (), {"stop_token_ids": (0,)})()
        self.sums = {}
        self.log = []
        self.peak_open = 0

    def open_sequences(self, n):
        slots = self.cache.open(n)
        for s in slots:
            self.sums[s] = 0
        self.peak_open = max(self.peak_open, self.cache.max_slots - self.cache.slots.n_free)
        self.log.append(("open", tuple(slots)))
        return slots

    def close_sequences(self, slots):
        self.log.append(("close", tuple(slots)))
        self.cache.close(slots)

    def step(self, entries):
        self.cache.reserve({e.slot: self.cache.length(e.slot) + len(e.tokens) for e in entries})
        rows = []
        self.log.append(("step", tuple((e.slot, len(e.tokens)) for e in entries)))
        for e in entries:
            for i, t in enumerate(e.tokens):
                self.sums[e.slot] += t
                if i in e.want:
                    pos = self.cache.length(e.slot) + i
                    row = torch.zeros(V)
                    row[(self.sums[e.slot] + pos) % V] = 1.0
                    rows.append(row)
            self.cache.advance(e.slot, len(e.tokens))
        return torch.stack(rows) if rows else torch.zeros((0, V))


def argmax_sampler(logits, sequence_indices, step, windows):
    return logits.argmax(-1).tolist()


def expected(prompt, n, stops=(0,), max_len=10 ** 9):
    seq, out = list(prompt), []
    while len(out) < n:
        tok = (sum(seq) + len(seq) - 1) % V
        if tok in stops:
            return out, FINISH_STOP
        out.append(tok)
        if len(out) >= n:
            return out, FINISH_LENGTH
        if len(seq) + 1 > max_len:
            return out, FINISH_CONTEXT
        seq.append(tok)
    return out, FINISH_LENGTH


def test_unequal_prompts_stops_and_early_ends():
    eng = ScriptedEngine()
    prompts = [[3, 4], [5], [7, 8, 9, 10], [11, 12, 13], [1] * 9, [2, 2], [6] * 20]
    stops = tuple(range(0, V, 7))
    res = generate(eng, prompts, max_new_tokens=12, sampler=argmax_sampler, stop_ids=stops)
    reasons = set()
    for p, r in zip(prompts, res):
        want, why = expected(p, 12, stops=stops)
        assert (r.tokens, r.finish_reason) == (want, why)
        assert not set(stops) & set(r.tokens)                      # a stop token is never emitted
        reasons.add(why)
    assert reasons == {FINISH_STOP, FINISH_LENGTH}
    assert eng.peak_open <= 3 and eng.cache.slots.n_free == 3 and eng.cache.free_pages() == [16]
    opens = [e for e in eng.log if e[0] == "open"]
    assert len(opens) == 3 and opens[1][1] == opens[0][1]          # the next batch starts in the same slots
    # the first step of a batch brings whole prompts of unequal lengths, later steps one token each
    first = next(e for e in eng.log if e[0] == "step")
    assert [n for _, n in first[1]] == [2, 1, 4]
    later = [e for e in eng.log if e[0] == "step" and e is not first][0]
    assert all(n == 1 for _, n in later[1])
    # sequences that end leave the batch: the number of sequences in a step never grows inside a batch
    prev = None
    for e in eng.log:
        if e[0] == "open":
            prev = None
        if e[0] == "step":
            assert prev is None or len(e[1]) <= prev
            prev = len(e[1])


def test_ignore_eos_and_custom_stop_ids():
    eng = ScriptedEngine()
    p = [[5]]
    full, _ = expected(p[0], 12, stops=())
    eng.plan.stop_token_ids = (full[5],)                          # the model's own stop token
    r = generate(eng, p, max_new_tokens=12, sampler=argmax_sampler)[0]
    assert r.tokens == full[:5] and r.finish_reason == FINISH_STOP
    assert generate(eng, p, max_new_tokens=12, sampler=argmax_sampler, ignore_eos=True)[0].tokens == full
    stop_at = full[3]
    r = generate(eng, p, max_new_tokens=12, sampler=argmax_sampler, stop_ids=[stop_at])[0]
    assert r.tokens == full[:full.index(stop_at)] and r.finish_reason == FINISH_STOP


def test_context_limit_ends_a_sequence():
    eng = ScriptedEngine(max_seq_len=PAGE_SIZE)
    prompt = [1] * (PAGE_SIZE - 2)
    r = generate(eng, [prompt], max_new_tokens=50, sampler=argmax_sampler, ignore_eos=True)[0]
    want, why = expected(prompt, 50, stops=(), max_len=PAGE_SIZE)
    assert why == FINISH_CONTEXT and (r.tokens, r.finish_reason) == (want, why)
    assert len(prompt) + len(r.tokens) == PAGE_SIZE + 1            # the last token was sampled, not run
    with pytest.raises(ValueError, match="longest"):
        generate(eng, [[1] * (PAGE_SIZE + 1)], sampler=argmax_sampler)
    with pytest.raises(ValueError, match="empty"):
        generate(eng, [[]], sampler=argmax_sampler)


def test_zero_new_tokens_and_stats():
    eng = ScriptedEngine()
    stats = GenerationStats()
    res = generate(eng, [[1, 2, 3], [4]], max_new_tokens=0, sampler=argmax_sampler, stats=stats)
    assert [r.tokens for r in res] == [[], []] and stats.prompt_tokens == 4 and stats.generated_tokens == 0
    ticks = iter(range(1000))
    stats = GenerationStats()
    generate(eng, [[5]], max_new_tokens=3, sampler=argmax_sampler, ignore_eos=True, stats=stats,
             clock=lambda: float(next(ticks)))
    assert stats.generated_tokens == 3 and stats.steps == 2 and stats.batches == 1
    assert "prefill: 1 tok" in stats.line() and "gen: 3 tok" in stats.line()


def test_plan_batches():
    assert plan_batches([10, 10, 10, 10, 10], 5, max_batch=2, max_tokens=10 ** 6, max_seq_len=4096) == [[0, 1], [2, 3], [4]]
    # pages: each request needs pages_for(prompt + new)
    assert plan_batches([60, 60, 60], 4, max_batch=8, max_tokens=2 * PAGE_SIZE, max_seq_len=4096) == [[0, 1], [2]]
    assert plan_batches([60, 60, 60], 5, max_batch=8, max_tokens=2 * PAGE_SIZE, max_seq_len=4096) == [[0], [1], [2]]
    with pytest.raises(ValueError, match="pages"):
        plan_batches([200], 5, max_batch=8, max_tokens=2 * PAGE_SIZE, max_seq_len=4096)


def test_sampling_params():
    assert SamplingParams().temperature == 0.8 and SamplingParams().top_k == 40 and SamplingParams().top_p == 0.95
    assert SamplingParams(temperature=0).greedy and not SamplingParams().penalized
    assert SamplingParams(repeat_penalty=1.1).penalized and not SamplingParams(repeat_penalty=1.1, repeat_last_n=0).penalized
    with pytest.raises(ValueError):
        SamplingParams(repeat_penalty=0)


def test_length_buckets_double():
    """A decode graph is captured for a bound on the lengths; the bound doubles, so a growing sequence needs few graphs."""
    from questwend_b200.engine.decode import length_bucket
    assert [length_bucket(n) for n in (1, 255, 256, 257, 1024, 1025, 5000)] == [256, 256, 256, 512, 1024, 2048, 8192]
    assert all(length_bucket(n) >= n for n in range(1, 3000, 7))
