"""The generation loop above the step function.

The reference's loop is for one sequence (cli/main.cpp:408-425): run the prompt,
then sample, stop if the token is a stop token (it is neither emitted nor counted),
emit, run the token, until ``max_tokens``.  Here the same loop runs for batches:
as many requests as fit start together with their whole prompts in one step; every
later step brings one token for each sequence that is still going; a sequence that
ends leaves the batch and gives its slot back at once; when a batch is done the next
requests start in the slots that came free.

The decisions (who starts, who ends and why, who goes on) use nothing of the
device, so they can be followed with any object that has ``open_sequences``,
``close_sequences``, ``step``, ``max_batch`` and ``cache``-like limits.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field

from ..cache.manager import pages_for
from ..sampling.params import GREEDY, SamplingParams
from ..sampling.sampler import DeviceSampler, PenaltyWindow
from .engine import StepEntry

FINISH_STOP = "stop"          # a stop token was sampled
FINISH_LENGTH = "length"      # max_new_tokens were emitted
FINISH_CONTEXT = "context"    # the sequence reached the longest length the cache allows


@dataclass
class GenerationResult:
    tokens: list = field(default_factory=list)
    finish_reason: str = ""
    prompt_tokens: int = 0


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    batches: int = 0
    steps: int = 0
    step_seconds: list = field(default_factory=list)    # every decode step's wall time, in order (its sum: decode_seconds)

    def line(self) -> str:
        """The reference's speed line (cli/main.cpp:427-432)."""
        pf = self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0
        gen = self.generated_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0
        return (f"[prefill: {self.prompt_tokens} tok in {self.prefill_seconds:.3f} s = {pf:.1f} tok/s | "
                f"gen: {self.generated_tokens} tok in {self.decode_seconds:.3f} s = {gen:.1f} tok/s]")


def plan_batches(prompt_lengths, max_new_tokens: int, max_batch: int, max_tokens: int, max_seq_len: int):
    """Cut the requests, in order, into batches that fit: at most ``max_batch`` sequences, and
    pages for every sequence at its longest (prompt + new tokens, capped by ``max_seq_len``)."""
    batches, cur, cur_pages = [], [], 0
    total_pages = pages_for(max_tokens)
    for i, n in enumerate(prompt_lengths):
        need = pages_for(min(n + max_new_tokens, max_seq_len))
        if need > total_pages:
            raise ValueError(f"request {i}: {n} prompt tokens and {max_new_tokens} new tokens need {need} pages; "
                             f"the cache has {total_pages} (max_tokens={max_tokens})")
        if cur and (len(cur) >= max_batch or cur_pages + need > total_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


class StepProfile:
    """Where a decode step's time goes, one line a step on ``out`` (the reference prints build / input / compute per
    token under QWEN_PROF, core/runtime.cpp:1769, 1821-1825):

      loop    the generation loop between two steps (stop tests, results, who goes on)
      host    preparing the step on the host (binding a changed batch, the step's tokens, page bookkeeping)
      launch  starting the step's work (a graph replay, or every kernel launch of a plain step)
      wait    waiting for the sampled ids
      device  the step on the device, between two CUDA events on the stream
    """

    def __init__(self, out=None, clock=time.perf_counter):
        import sys
        self.out = out if out is not None else sys.stderr
        self.clock = clock
        self.rows: list = []
        self._last_end = None
        self._events = None

    def begin(self):
        import torch
        t = self.clock()
        self._loop = 0.0 if self._last_end is None else t - self._last_end
        self._t0 = t
        self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))

    def launching(self):
        self._t1 = self.clock()
        self._events[0].record()

    def launched(self):
        self._events[1].record()
        self._t2 = self.clock()

    def end(self, step: int, batch: int, how: str):
        t3 = self.clock()
        self._events[1].synchronize()
        row = {"step": step, "batch": batch, "how": how, "loop_ms": self._loop * 1e3, "host_ms": (self._t1 - self._t0) * 1e3,
               "launch_ms": (self._t2 - self._t1) * 1e3, "wait_ms": (t3 - self._t2) * 1e3,
               "device_ms": self._events[0].elapsed_time(self._events[1])}
        self.rows.append(row)
        print("[prof] step=%d batch=%d %s loop=%.3f host=%.3f launch=%.3f wait=%.3f device=%.3f ms" % (
            step, batch, how, row["loop_ms"], row["host_ms"], row["launch_ms"], row["wait_ms"], row["device_ms"]),
            file=self.out)
        self._last_end = self.clock()


class _PlainStepper:
    """Decode steps through ``engine.step`` and a sampler callable."""

    def __init__(self, engine, sampler, slot_of, windows, profile=None):
        self.engine, self.sampler, self.slot_of, self.windows = engine, sampler, slot_of, windows
        self.profile = profile

    def run(self, active, tokens, step):
        prof = self.profile
        if prof:
            prof.begin()
        entries = [StepEntry(self.slot_of[i], [t], [0]) for i, t in zip(active, tokens)]
        if prof:
            prof.launching()
        logits = self.engine.step(entries)
        if prof:
            prof.launched()
        ids = self.sampler(logits, active, step, [self.windows[i] for i in active])
        if prof:
            prof.end(step, len(active), "plain")
        return ids


class _GraphStepper:
    """Decode steps replayed from CUDA graphs (``DecodeRunner``); rebinds when the batch changes."""

    def __init__(self, engine, sampling, seed, slot_of, windows, profile=None):
        self.engine, self.sampling, self.seed = engine, sampling, seed
        self.slot_of, self.windows = slot_of, windows
        self.bound = None
        self.runner = None
        self.profile = profile

    def run(self, active, tokens, step):
        prof = self.profile
        if prof:
            prof.begin()
        if self.bound != active:
            self.runner = self.engine.decode_runner(len(active), self.sampling)
            self.runner.bind([self.slot_of[i] for i in active], tokens, active, step,
                             [self.windows[i] for i in active], seed=self.seed)
            self.bound = list(active)
        if prof:
            self.runner.profile = prof
        self.runner.step(host_tokens=tokens)
        ids = self.runner.read_sampled()
        if prof:
            self.runner.profile = None
            prof.end(step, len(active), self.runner.last_step_how)
        return ids


def generate(engine, prompts, max_new_tokens: int = 128, sampling: SamplingParams = GREEDY,
             stop_ids=None, ignore_eos: bool = False, sampler=None, stats: GenerationStats | None = None,
             clock=time.perf_counter, use_graph: bool = True, profile=None) -> list[GenerationResult]:
    """Generate for every prompt (a list of token ids each).

    stop_ids    tokens that end a sequence; default: the model's own (``eos_token_id``)
    ignore_eos  never stop on a token (benchmarks)
    sampler     ``(logits, sequence_indices, step, windows) -> list of ids``; default: the device sampler
    use_graph   replay decode steps from CUDA graphs (needs the default sampler)
    profile     a ``StepProfile``, or True for one that prints to stderr: a line per decode step that says where its
                time went (also switched on by the environment variable QWB200_PROF=1)
    """
    if profile is None and os.environ.get("QWB200_PROF", "0") not in ("", "0"):
        profile = True
    if profile is True:
        profile = StepProfile()
    prompts = [list(p) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            raise ValueError(f"request {i}: the prompt is empty")
        if len(p) > engine.cache.max_seq_len:
            raise ValueError(f"request {i}: the prompt has {len(p)} tokens; the longest sequence allowed is "
                             f"{engine.cache.max_seq_len}")
    if stop_ids is None:
        stop_ids = tuple(getattr(engine.plan, "stop_token_ids", ()))
    stops = frozenset() if ignore_eos else frozenset(stop_ids)
    graph_path = use_graph and sampler is None and hasattr(engine, "decode_runner")
    if sampler is None:
        sampler = DeviceSampler(sampling, engine.device)
    stats = stats if stats is not None else GenerationStats()
    results = [GenerationResult(prompt_tokens=len(p)) for p in prompts]
    max_seq_len = engine.cache.max_seq_len

    max_batch = engine.max_batch
    held = getattr(engine.cache, "slots", None)
    if held is not None:                    # slots that someone else holds meanwhile are not this call's to plan with
        max_batch = max(1, min(max_batch, held.n_free))
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, max_batch,
                              engine.cache.max_tokens, max_seq_len):
        stats.batches += 1
        slots = engine.open_sequences(len(batch))
        slot_of = dict(zip(batch, slots))
        windows = {i: PenaltyWindow(sampling, prompts[i]) for i in batch}
        length = {i: len(prompts[i]) for i in batch}
        active = list(batch)
        stepper = (_GraphStepper(engine, sampling, sampler.seed, slot_of, windows, profile) if graph_path
                   else _PlainStepper(engine, sampler, slot_of, windows, profile))
        try:
            t0 = clock()
            want_last = max_new_tokens > 0
            logits = engine.step([StepEntry(slot_of[i], prompts[i], [len(prompts[i]) - 1] if want_last else [])
                                  for i in active])
            ids = sampler(logits, active, 0, [windows[i] for i in active]) if want_last else []
            stats.prefill_seconds += clock() - t0
            stats.prompt_tokens += sum(len(prompts[i]) for i in active)
            step = 1
            while want_last and active:
                going, done = [], []
                for i, tok in zip(active, ids):
                    tok = int(tok)
                    if tok in stops:                         # not emitted, not counted
                        results[i].finish_reason = FINISH_STOP
                        done.append(i)
                        continue
                    results[i].tokens.append(tok)
                    windows[i].accept(tok)
                    stats.generated_tokens += 1
                    if len(results[i].tokens) >= max_new_tokens:
                        results[i].finish_reason = FINISH_LENGTH
                        done.append(i)
                    elif length[i] + 1 > max_seq_len:        # no room to run this token
                        results[i].finish_reason = FINISH_CONTEXT
                        done.append(i)
                    else:
                        going.append(i)
                if done:
                    engine.close_sequences([slot_of.pop(i) for i in done])
                active = going
                if not active:
                    break
                t0 = clock()
                ids = stepper.run(active, [results[i].tokens[-1] for i in active], step)
                took = clock() - t0
                stats.decode_seconds += took
                stats.step_seconds.append(took)
                for i in active:
                    length[i] += 1
                step += 1
                stats.steps += 1
            if graph_path:
                engine.check_kernels()            # the steps replayed from graphs are checked once a batch (plain steps each)
        finally:
            if slot_of:
                engine.close_sequences(list(slot_of.values()))
        for i in batch:
            if not results[i].finish_reason:
                results[i].finish_reason = FINISH_LENGTH
    return results
