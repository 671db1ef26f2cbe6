"""Decode steps from a CUDA graph.

After the prompts have run, every step is the same work on one more token per
sequence.  ``DecodeRunner`` keeps that step's inputs in fixed device buffers
(token ids, positions, lengths, page tables, the sampler's state), captures
"model step -> sample -> advance" once per batch size and attention-grid bucket,
and replays it.  The step inside the graph is the same ``Model.forward`` that
``Engine.step`` runs; only its inputs come from the fixed buffers.  The host keeps
the cache's bookkeeping (it knows every length without asking the device) and
refreshes the page tables when a sequence needs a new page.

The reference does the same for its single sequence: a persistent graph whose
write position and mask are inputs, rebuilt only when the key count crosses a
bucket of 32 (core/runtime.cpp:1768-1829), replayed as a CUDA graph inside ggml.
"""
from __future__ import annotations

import gc

import numpy as np
import torch

from ..kernels import ops
from ..parts.base import StepContext
from ..sampling.params import SamplingParams


MIN_BUCKET = 256
N_SCALARS = 4               # int32 words before the rows of the state buffer: seed (two words), step, one unused
N_ROWS = 7
GRAPH_AFTER = 2             # plain steps at a batch size and length bound before a graph is captured for them


def length_bucket(n_tokens: int) -> int:
    """The bound on the sequences' length that a graph is captured for: the next power of two (at least 256).
    The attention kernels size their grid and scratch by it and let the blocks beyond a sequence's keys return at once,
    so a generous bound costs little, and a sequence that grows needs a new graph only when its length doubles."""
    return max(MIN_BUCKET, 1 << max(0, n_tokens - 1).bit_length())


class DecodeRunner:
    """Fixed buffers and graphs for decode steps of ``batch`` sequences with one sampling setup."""

    def __init__(self, engine, batch: int, sampling: SamplingParams, use_graph: bool = True):
        self.engine = engine
        self.B = B = batch
        self.sampling = sampling
        self.use_graph = use_graph
        if GRAPH_AFTER < 1:
            raise ValueError("a graph is captured only after a plain step has loaded the kernels")
        dev = engine.device
        cache = engine.cache
        # One int32 buffer, one copy per bind: [seed low, seed high, step, unused] then seven rows of B:
        # token_ids, tok_pos, pos0, seq_len, sequence_index, n_seen, slot ids.  The seed, the step counter and the
        # slot ids live on the device, so a captured graph holds none of them: it serves every batch of this size.
        self.state_flat = torch.zeros((N_SCALARS + N_ROWS * B,), dtype=torch.int32, device=dev)
        self.seed_word = self.state_flat[0:2].view(torch.int64)
        self.step_counter = self.state_flat[2:3]
        self.state = self.state_flat[N_SCALARS:].view(N_ROWS, B)
        (self.token_ids, self.tok_pos, self.pos0, self.seq_len, self.seq_index, self.n_seen,
         self.slot_ids) = self.state.unbind(0)
        self.tok_seq = torch.arange(B, dtype=torch.int32, device=dev)
        self.cu_seqlens = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.rows = torch.arange(B, dtype=torch.int32, device=dev)
        self.sampled = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.window = sampling.repeat_last_n if sampling.penalized else 0
        self.recent = (torch.full((B, self.window), -1, dtype=torch.int32, device=dev) if self.window else None)
        self.tables = {g: torch.zeros((B, cache.table_width), dtype=torch.int32, device=dev)
                       for g in range(cache.n_groups())}
        self.tables_host = {g: torch.zeros((B, cache.table_width), dtype=torch.int32).pin_memory()
                            for g in range(cache.n_groups())}
        self.state_host = torch.zeros((N_SCALARS + N_ROWS * B,), dtype=torch.int32).pin_memory()
        self._state_np = self.state_host.numpy()
        self.tokens_host = torch.zeros((B,), dtype=torch.int32).pin_memory()
        self.sampled_host = torch.zeros((B,), dtype=torch.int32).pin_memory()
        self._tokens_np = self.tokens_host.numpy()      # the same pinned memory, written and read without a tensor op
        self._sampled_np = self.sampled_host.numpy()
        self._sampled_on_host = False                   # the last step copied its ids to the host itself
        self._copied = None                             # event: the pinned buffers' last copies to the device are done
        self.graphs: dict = {}                          # (length bound, with host copies) -> graph
        self._pool = None           # the graphs run one at a time: they share one pool of memory
        self.slots: list = []
        self._pages_seen: list = []
        self._room = 0              # steps that need no new page and no other graph (see step)
        self._graph = {}            # with host copies or not -> the graph for the steps in this room
        self._plain_steps: dict = {}    # length bound -> plain steps run so far
        self.launches_per_step = 0
        self.profile = None         # a StepProfile while someone wants to know where a step's time goes
        self.last_step_how = ""     # "graph" or "plain"

    # ------------------------------------------------------------------ binding a batch
    def bind(self, slots, tokens, sequence_indices, step: int, windows=None, seed: int = 0) -> None:
        """Point the buffers at these sequences: ``tokens`` are the next inputs (one each); ``seed`` and ``step`` key the
        sampler's random streams.  One copy from pinned memory, no wait: the copy is ordered before the next step on the
        stream, and the pinned buffer is written again only after the copy has been seen to finish."""
        assert len(slots) == self.B
        B = self.B
        cache = self.engine.cache
        self.slots = list(slots)
        lens = [cache.length(s) for s in slots]
        if self._copied is not None:
            self._copied.synchronize()
        h = self._state_np
        seed &= (1 << 64) - 1
        h[0:2] = np.array([seed & 0xFFFFFFFF, seed >> 32], dtype=np.uint32).view(np.int32)
        h[2] = step
        rows = h[N_SCALARS:].reshape(N_ROWS, B)
        rows[0] = tokens
        rows[1] = lens
        rows[2] = lens
        rows[3] = rows[1] + 1
        rows[4] = sequence_indices
        rows[5] = 0
        rows[6] = slots
        if self.window:
            recent = [w.row() for w in windows]
            rows[5] = [sum(1 for t in r if t >= 0) for r in recent]
            self.recent.copy_(torch.tensor(recent, dtype=torch.int32))
        self.state_flat.copy_(self.state_host, non_blocking=True)
        self._copied = torch.cuda.Event()
        self._copied.record()
        self._pages_seen = [None] * cache.n_groups()
        self._room = 0

    def set_tokens(self, tokens) -> None:
        """This step's input tokens from the host (pinned memory, one copy)."""
        self.tokens_host.copy_(torch.as_tensor(tokens, dtype=torch.int32))
        self.token_ids.copy_(self.tokens_host, non_blocking=True)

    # ------------------------------------------------------------------ one step
    def _context(self, max_len_bucket: int) -> StepContext:
        return StepContext(n_tokens=self.B, n_seqs=self.B, token_ids=self.token_ids, tok_seq=self.tok_seq,
                           tok_pos=self.tok_pos, cu_seqlens=self.cu_seqlens, pos0=self.pos0, seq_len=self.seq_len,
                           slots=self.slot_ids, max_new=1, max_len=max_len_bucket, single_token=True,
                           page_tables=self.tables, host_slots=None)

    def _forward_and_sample(self, max_len_bucket: int) -> None:
        eng, p = self.engine, self.sampling
        logits = eng.model.forward(self._context(max_len_bucket), eng.unit_caches, self.rows)
        ops.sample(logits, p.temperature, top_k=p.top_k, top_p=p.top_p, seed=0, seed_from=self.seed_word,
                   sequence_index=self.seq_index, step=0, step_add=self.step_counter, recent=self.recent,
                   repeat_penalty=p.repeat_penalty, presence_penalty=p.presence_penalty,
                   frequency_penalty=p.frequency_penalty, out=self.sampled)

    def _advance(self) -> None:
        ops.decode_advance(self.sampled, self.token_ids, self.tok_pos, self.pos0, self.seq_len,
                           step_counter=self.step_counter, recent=self.recent,
                           n_seen=self.n_seen if self.window else None)

    def _capture(self, bucket: int, host_copies: bool):
        # Plain steps at this batch size and length bound came before (GRAPH_AFTER): they loaded the kernels, set their
        # attributes and let the few-rows products settle their choices.  No extra run here: a mixer with state of its
        # own would count a token twice.
        torch.cuda.current_stream().synchronize()
        g = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES[0]
        # No garbage collection while the stream is capturing: an unreachable engine's graphs would be destroyed
        # in the middle of it, which CUDA refuses during a capture and which invalidates the capture.
        collect_again = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            if self._pool is None:
                self._pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(g, pool=self._pool):
                if host_copies:         # the step's tokens come from pinned host memory and its ids go back there:
                    self.token_ids.copy_(self.tokens_host, non_blocking=True)      # two copy nodes of the graph
                self._forward_and_sample(bucket)
                self._advance()
                if host_copies:
                    self.sampled_host.copy_(self.sampled, non_blocking=True)
        finally:
            if collect_again:
                gc.enable()
        self.launches_per_step = ops.LAUNCHES[0] - before
        return g

    def step(self, host_tokens=None) -> None:
        """Run one decode step for the bound sequences; the sampled ids land in ``self.sampled``
        and become the next inputs.  ``host_tokens``: this step's input tokens as the host knows them; the step
        then copies them in from pinned memory and copies its ids out to pinned memory (``read_sampled`` only
        waits), inside the graph when it is replayed.  None: the inputs are on the device already."""
        cache = self.engine.cache
        host_copies = host_tokens is not None
        if host_copies:
            self._tokens_np[:] = host_tokens
        if self._room <= 0:
            # A sequence may need a page, or the longest one leaves the graph's bucket: look, and count the steps
            # until either can happen again.  Nothing else changes between the steps of a bound batch.
            lengths = [cache.length(s) for s in self.slots]
            cache.reserve({s: n + 1 for s, n in zip(self.slots, lengths)})
            room = cache.max_seq_len - max(lengths)          # reserve() refuses a longer sequence: let it look then
            for g in range(cache.n_groups()):
                counts = [len(cache._groups[g].pages[s]) for s in self.slots]
                if counts != self._pages_seen[g]:
                    self._pages_seen[g] = counts
                    if self._copied is not None:
                        self._copied.synchronize()
                    self.tables_host[g].numpy()[:] = cache.page_table_host(g, self.slots)
                    self.tables[g].copy_(self.tables_host[g], non_blocking=True)
                    self._copied = torch.cuda.Event()
                    self._copied.record()
                room = min(room, min(c * ops.PAGE_SIZE - n for c, n in zip(counts, lengths)))
            self._bucket = length_bucket(max(lengths) + 1)
            self._room = min(room, self._bucket - max(lengths))
            self._graph = {}
        self._room -= 1
        prof = self.profile
        with torch.cuda.device(self.engine.device):
            graph = self._graph.get(host_copies)
            if self.use_graph and graph is None:
                key = (self._bucket, host_copies)
                graph = self.graphs.get(key)
                if graph is None and self._plain_steps.get(self._bucket, 0) >= GRAPH_AFTER:
                    # a capture costs about two steps: it pays only for a batch that stays (a batch whose sequences
                    # end one after the other passes through many sizes for a step or two each)
                    graph = self.graphs[key] = self._capture(self._bucket, host_copies)
                self._graph[host_copies] = graph
            if prof:
                prof.launching()
            self.last_step_how = "graph" if graph is not None else "plain"
            if graph is not None:
                graph.replay()
            else:
                if host_copies:
                    self.token_ids.copy_(self.tokens_host, non_blocking=True)
                before = ops.LAUNCHES[0]
                self._forward_and_sample(self._bucket)
                self._advance()
                self.launches_per_step = ops.LAUNCHES[0] - before
                self._plain_steps[self._bucket] = self._plain_steps.get(self._bucket, 0) + 1
                if host_copies:
                    self.sampled_host.copy_(self.sampled, non_blocking=True)
            if prof:
                prof.launched()
        self._sampled_on_host = host_copies
        for s in self.slots:
            cache.advance(s, 1)
        self.engine.steps_run += 1

    def read_sampled(self) -> list:
        """The ids sampled by the last step, on the host (waits for the step; copies first if the step did not)."""
        if not self._sampled_on_host:
            self.sampled_host.copy_(self.sampled, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._sampled_np.tolist()
