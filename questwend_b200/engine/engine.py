"""The engine: a model, its cache, and the one step function.

``step`` takes a batch of sequences, each with its next tokens (a whole prompt, or
one token), runs exactly those tokens as one packed batch against the cache that
earlier steps left, and returns the logits at the places asked for.  There is no
padding anywhere: sequences of unequal length are packed end to end, and the
kernels take each sequence's own start and length.

The reference's counterpart is ``Runtime::decode`` for one sequence
(core/runtime.cpp:3020-3203 for a prompt, :1768-1829 for one token), which
returns the last position's logits only (core/runtime.h:52-54).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache.manager import CacheManager, pages_for
from ..config.base import ModelConfig
from ..config.registry import get_architecture, load_config
from ..kernels import build as kernel_build
from ..kernels import ops
from ..kernels.ops import PAGE_SIZE
from ..parts.base import Runtime, StepContext
from ..parts.linear import require_true_fp32
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors
from .model import Model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class EngineError(RuntimeError):
    pass


@dataclass
class StepEntry:
    """One sequence's part of a step: its slot, its next tokens, and the places among
    these tokens (0-based) whose logits are wanted."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)


def _require_cuda(device: torch.device) -> None:
    if device.type != "cuda":
        raise EngineError(f"the engine runs on a CUDA device only, got '{device}' (there is no CPU path)")
    if not torch.cuda.is_available():
        raise EngineError("no CUDA device is available; the engine has no CPU path")
    major, minor = torch.cuda.get_device_capability(device)
    if (major, minor) != (10, 0):
        raise EngineError(f"the kernels are built for sm_100a (B200); this device is sm_{major}{minor}")


def build_step_context(cache: CacheManager, entries: list, vocab_size: int, device) -> tuple[StepContext, torch.Tensor]:
    """Pack one step's entries for the device: reserves cache pages for the new tokens (or raises and
    changes nothing), and returns the context and the packed rows whose logits are wanted."""
    if not entries:
        raise EngineError("a step needs at least one sequence")
    slots = [e.slot for e in entries]
    if len(set(slots)) != len(slots):
        raise EngineError(f"a slot appears twice in one step: {slots}")
    B = len(entries)
    n_new = []
    for e in entries:
        if len(e.tokens) == 0:
            raise EngineError(f"slot {e.slot}: a step must bring at least one token for each sequence")
        n_new.append(len(e.tokens))
    T = sum(n_new)
    pos0 = [cache.length(s) for s in slots]

    # one packed int32 buffer, one copy to the device
    n_want = sum(len(e.want) for e in entries)
    offs = np.cumsum([0, T, T, T, B + 1, B, B, B, n_want])
    buf = np.empty(offs[-1], dtype=np.int32)
    ids, tok_seq, tok_pos, cu, p0, slen, slot_a, want = (buf[offs[i]:offs[i + 1]] for i in range(8))
    t = 0
    w = 0
    for b, e in enumerate(entries):
        n = n_new[b]
        try:
            ids[t:t + n] = e.tokens
        except (TypeError, ValueError, OverflowError):
            raise EngineError(f"slot {e.slot}: token ids must be integers") from None
        tok_seq[t:t + n] = b
        tok_pos[t:t + n] = np.arange(pos0[b], pos0[b] + n)
        cu[b] = t
        for i in e.want:
            if not 0 <= i < n:
                raise EngineError(f"slot {e.slot}: wanted place {i} is outside this step's {n} tokens")
            want[w] = t + i
            w += 1
        t += n
    cu[B] = T
    if T and (ids.min() < 0 or ids.max() >= vocab_size):
        bad = int(ids[(ids < 0) | (ids >= vocab_size)][0])
        raise EngineError(f"token id {bad} is outside the vocabulary of {vocab_size}")
    p0[:] = pos0
    slen[:] = [p + n for p, n in zip(pos0, n_new)]
    slot_a[:] = slots
    cache.reserve({s: p + n for s, p, n in zip(slots, pos0, n_new)})     # after every check: a refused step holds nothing
    dev = torch.from_numpy(buf).to(device)
    parts = [dev[offs[i]:offs[i + 1]] for i in range(8)]
    tables = {}
    for gid in range(cache.n_groups()):
        tables[gid] = torch.from_numpy(cache.page_table_host(gid, slots)).to(device)
    ctx = StepContext(n_tokens=T, n_seqs=B, token_ids=parts[0], tok_seq=parts[1], tok_pos=parts[2],
                      cu_seqlens=parts[3], pos0=parts[4], seq_len=parts[5], slots=parts[6],
                      max_new=max(n_new), max_len=int(max(slen)), single_token=all(n == 1 for n in n_new),
                      page_tables=tables, host_slots=slots)
    return ctx, parts[7]


class Engine:
    """Build with ``Engine.from_folder`` or ``Engine.from_config``.

    max_tokens   the most tokens live sequences hold together (each rounded up to pages of 64)
    max_seq_len  the longest single sequence (default: max_tokens, capped by the model's trained length)
    max_batch    the most sequences alive at once (default: as many as could each hold one page, up to 256)
    """

    def __init__(self, config: ModelConfig, weights: dict, dtype: torch.dtype, device: torch.device,
                 max_tokens: int, max_seq_len: int | None = None, max_batch: int | None = None):
        self.config = config
        self.dtype = dtype
        self.device = device
        if dtype == torch.float32:
            require_true_fp32()
        arch = get_architecture(config.architecture)
        self.plan = arch.plan(config)
        self.runtime = Runtime(device, dtype)
        self.model = Model(self.plan, self.runtime)
        kernel_build.compile_modules(self.model.kernel_modules())
        self.model.bind(weights)
        self.vocab_size = self.plan.vocab_size
        if max_seq_len is None:
            max_seq_len = max_tokens
            if self.plan.max_position:
                max_seq_len = min(max_seq_len, self.plan.max_position)
        max_seq_len = min(max_seq_len, pages_for(max_tokens) * PAGE_SIZE)
        if max_batch is None:
            max_batch = max(1, min(256, pages_for(max_tokens)))
        self.max_batch = max_batch
        self.cache = CacheManager(self.model.cache_units(), max_tokens, max_batch, max_seq_len, dtype, device)
        self.unit_caches = [self.cache.unit_cache(i) for i in range(len(self.model.schedule))]
        self.steps_run = 0
        self._runners: dict = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        device = torch.device(device)
        _require_cuda(device)
        dtype = DTYPES[dtype]
        config = load_config(model_dir)
        plan = get_architecture(config.architecture).plan(config)
        weights = load_tensors(model_dir, plan.manifest(), dtype, device)
        return cls(config, weights, dtype, device, **kw)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        """Random weights drawn on the device (the values differ from a folder written with the same seed)."""
        device = torch.device(device)
        _require_cuda(device)
        dtype = DTYPES[dtype]
        plan = get_architecture(config.architecture).plan(config)
        weights = random_tensors(plan.manifest(), seed, dtype, device=device, vector_dtype=torch.float32)
        return cls(config, weights, dtype, device, **kw)

    # ------------------------------------------------------------------ sequences
    def open_sequences(self, count: int) -> list[int]:
        return self.cache.open(count)

    def close_sequences(self, slots) -> None:
        self.cache.close(slots)

    # ------------------------------------------------------------------ the step
    def build_context(self, entries: list[StepEntry]) -> tuple[StepContext, torch.Tensor]:
        return build_step_context(self.cache, entries, self.vocab_size, self.device)

    @torch.no_grad()
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; returns float32 logits [wanted, vocab] on the device, in the
        order of the entries and of each entry's ``want``."""
        with torch.cuda.device(self.device):
            ctx, want_rows = self.build_context(entries)
            logits = self.model.forward(ctx, self.unit_caches, want_rows)
            self.check_kernels()
        for e in entries:
            self.cache.advance(e.slot, len(e.tokens))
        self.steps_run += 1
        return logits

    def check_kernels(self) -> None:
        """Raise if a kernel with bounded waits (the TMA-fed products, the tcgen05 attention) gave one up since the last
        check: its result is then not valid.  Reads one int from the device, so it waits for the work queued so far."""
        if self.dtype == torch.bfloat16:
            with torch.cuda.device(self.device):
                ops.gemm_tc_check(self.device)

    def decode_runner(self, batch: int, sampling, use_graph: bool = True):
        """The fixed buffers and CUDA graphs for decode steps of ``batch`` sequences (made once, kept).  The sampling
        options without the seed key it: the seed lives on the device and is given with ``bind``."""
        import dataclasses
        from .decode import DecodeRunner
        sampling = dataclasses.replace(sampling, seed=0)
        key = (batch, sampling, use_graph)
        runner = self._runners.get(key)
        if runner is None:
            if len(self._runners) >= 16:             # graphs hold memory: drop the oldest
                self._runners.pop(next(iter(self._runners)))
            runner = self._runners[key] = DecodeRunner(self, batch, sampling, use_graph)
        return runner

    # ------------------------------------------------------------------ facts
    def describe(self) -> dict:
        n_params = sum(int(np.prod(t.shape)) for t in self.model.tensors() if not (t.optional or t.ignored))
        return {"architecture": self.config.architecture, "dtype": str(self.dtype).replace("torch.", ""),
                "parameters": n_params, "cache_bytes": self.cache.bytes_held(),
                "max_tokens": self.cache.max_tokens, "max_seq_len": self.cache.max_seq_len,
                "max_batch": self.max_batch, "page_size": PAGE_SIZE, "layers": len(self.plan.layers),
                "schedule": len(self.plan.schedule), "cache_groups": self.cache.n_groups()}
