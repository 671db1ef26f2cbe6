"""The sampler that generation uses: one device kernel call per step.

The reference samples on the host from a copy of the logits, with one
``std::mt19937`` per process (core/sampler.cpp:38-109).  Here the logits stay on the
device; each sequence has a random stream of its own, keyed by (seed, the sequence's
index in the call, how many tokens it has sampled), so what a sequence draws does
not depend on what else is in its batch.
"""
from __future__ import annotations

import os
from collections import deque

import torch

from ..kernels import ops
from .params import SamplingParams


class PenaltyWindow:
    """The last ``repeat_last_n`` tokens of a sequence: the prompt's tail, then what was
    generated (``prime`` and ``accept``, core/sampler.cpp:20-36)."""

    def __init__(self, params: SamplingParams, prompt):
        self.on = params.penalized
        self.n = params.repeat_last_n
        self.recent = deque(prompt[-self.n:] if self.on else [], maxlen=max(self.n, 1))

    def accept(self, token: int) -> None:
        if self.on:
            self.recent.append(token)

    def row(self) -> list[int]:
        r = list(self.recent)
        return r + [-1] * (self.n - len(r))


class DeviceSampler:
    def __init__(self, params: SamplingParams, device):
        self.params = params
        self.device = device
        seed = params.seed
        if seed == 0 and not params.greedy:
            seed = int.from_bytes(os.urandom(8), "little") or 1
        self.seed = seed

    def __call__(self, logits: torch.Tensor, sequence_indices: list[int], step: int,
                 windows: list[PenaltyWindow] | None = None) -> list[int]:
        """Token ids for the rows of ``logits`` [B, V] (float32, on the device)."""
        p = self.params
        recent = None
        if p.penalized and windows is not None:
            recent = torch.tensor([w.row() for w in windows], dtype=torch.int32, device=logits.device)
        seq = torch.tensor(sequence_indices, dtype=torch.int32, device=logits.device)
        ids = ops.sample(logits, p.temperature, top_k=p.top_k, top_p=p.top_p, seed=self.seed,
                         sequence_index=seq, step=step, recent=recent, repeat_penalty=p.repeat_penalty,
                         presence_penalty=p.presence_penalty, frequency_penalty=p.frequency_penalty)
        return ids.tolist()
