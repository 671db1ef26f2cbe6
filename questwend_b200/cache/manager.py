"""The cache: a slot for each live sequence, keys and values for each scheduled layer run,
and per-sequence state of fixed size.

The reference holds one sequence: per layer a ``[n_ctx, Hkv*hd]`` K and V tensor and a
single ``n_past`` (core/runtime.cpp:113-114, 166, 503-504), plus fixed-size recurrent
state for layers that have it (:115-116, 493-494), zeroed at start (:614-630).  Here:

* A **slot** stands for one sequence: its length, its pages, its row in every state
  tensor.  Slots are handed out when a batch starts and given back when a sequence
  ends; a slot that was given back is handed out again.
* Keys and values live in **pages** of ``PAGE_SIZE`` tokens.  Layer runs whose mixers
  ask for the same ``KVSpec`` (heads, head size, window) form a **group**; each group
  has storage of its own, ``[units, pages, Hkv, PAGE_SIZE, hd]`` for K and for V, a
  page pool of its own and a page table of its own (one page id is valid in every
  unit of its group).  ``max_tokens`` sizes each pool: the most tokens that live
  sequences may hold together, each sequence's count rounded up to whole pages.
* The pools are zeroed once, when they are made.  Nothing is zeroed when a page or
  slot is handed out again: kernels never use what lies beyond a sequence's length
  (the tensor-core kernels multiply it by probability 0, so it must be finite: it is
  zero or an earlier sequence's keys and values).  State tensors are the exception (a recurrent state
  starts from zero), so a slot's state rows are zeroed when the slot is handed out.

All bookkeeping is on the host; the device sees page tables and lengths.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..kernels.ops import PAGE_SIZE
from ..parts.base import KVSpec, StateSpec, UnitCache


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """Not enough free pages or slots; nothing was changed."""


class FreeList:
    """Ids 0..n-1, each either free or held.  Lowest free id first, so ids are used again soon."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))      # pop() gives the lowest
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, count: int = 1) -> list[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}s wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            self._held[i] = True
        return out

    def give_back(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if not 0 <= i < self.n:
                raise CacheError(f"{self.what} {i} does not exist")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} is given back but is not held")
            self._held[i] = False
        self._free.extend(ids)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE_SIZE - 1) // PAGE_SIZE


@dataclass
class _KVGroup:
    spec: KVSpec
    units: list            # schedule indices that own storage here
    pool: FreeList
    k: torch.Tensor        # [units, pages, Hkv, PAGE_SIZE, hd]
    v: torch.Tensor
    pages: dict            # slot -> list of page ids, in order


@dataclass
class _StateUnit:
    spec: StateSpec
    storage: torch.Tensor  # [max_slots, *shape]


class CacheManager:
    """``units``: one ``(kv_spec | None, state_spec | None, cache_of | None)`` per scheduled run."""

    def __init__(self, units, max_tokens: int, max_slots: int, max_seq_len: int, dtype: torch.dtype,
                 device: torch.device | str):
        if max_tokens <= 0 or max_slots <= 0 or max_seq_len <= 0:
            raise CacheError(f"cache sizes must be positive: max_tokens={max_tokens} max_slots={max_slots} "
                             f"max_seq_len={max_seq_len}")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_tokens = max_tokens
        self.max_slots = max_slots
        self.max_seq_len = max_seq_len
        self.n_pages = pages_for(max_tokens)
        self.table_width = pages_for(max_seq_len)
        self.slots = FreeList(max_slots, "slot")
        self.lengths = [0] * max_slots
        self._groups: list[_KVGroup] = []
        self._unit_group: dict[int, tuple[int, int]] = {}     # schedule index -> (group id, index in group)
        self._unit_state: dict[int, _StateUnit] = {}
        self._cache_of: dict[int, int] = {}

        by_spec: dict[KVSpec, list[int]] = {}
        for i, (kv, state, cache_of) in enumerate(units):
            if cache_of is not None:
                self._cache_of[i] = cache_of
                continue
            if kv is not None:
                by_spec.setdefault(kv, []).append(i)
            if state is not None:
                storage = torch.zeros((max_slots, *state.shape), dtype=state.dtype, device=self.device)
                self._unit_state[i] = _StateUnit(state, storage)
        for gid, (spec, members) in enumerate(by_spec.items()):
            shape = (len(members), self.n_pages, spec.n_kv_heads, PAGE_SIZE, spec.head_dim)
            # zeroed once (the reference zeroes its cache too, core/runtime.cpp:614-630): a page's unused tail is
            # multiplied by probability 0 in the tensor-core kernels and must hold finite numbers
            k = torch.zeros(shape, dtype=dtype, device=self.device)
            v = torch.zeros(shape, dtype=dtype, device=self.device)
            self._groups.append(_KVGroup(spec, members, FreeList(self.n_pages, "page"), k, v, {}))
            for j, u in enumerate(members):
                self._unit_group[u] = (gid, j)

    # ------------------------------------------------------------------ what layers see
    def n_groups(self) -> int:
        return len(self._groups)

    def group_spec(self, gid: int) -> KVSpec:
        return self._groups[gid].spec

    def unit_cache(self, unit: int) -> UnitCache:
        owner = self._cache_of.get(unit, unit)
        writable = owner == unit
        gid = k = v = state = None
        if owner in self._unit_group:
            gid, j = self._unit_group[owner]
            k, v = self._groups[gid].k[j], self._groups[gid].v[j]
        if owner in self._unit_state:
            state = self._unit_state[owner].storage
        return UnitCache(gid, k, v, state, writable)

    def bytes_held(self) -> int:
        n = 0
        for g in self._groups:
            n += (g.k.numel() + g.v.numel()) * g.k.element_size()
        for s in self._unit_state.values():
            n += s.storage.numel() * s.storage.element_size()
        return n

    # ------------------------------------------------------------------ slots
    def open(self, count: int = 1) -> list[int]:
        """Hand out ``count`` slots with length 0, no pages and zeroed state."""
        slots = self.slots.take(count)
        for s in slots:
            self.lengths[s] = 0
            for g in self._groups:
                g.pages[s] = []
        if self._unit_state and slots:
            idx = torch.tensor(slots, dtype=torch.long, device=self.device)
            for st in self._unit_state.values():
                st.storage.index_fill_(0, idx, 0)
        return slots

    def close(self, slots) -> None:
        """Give slots and everything they hold back."""
        slots = list(slots)
        for s in slots:
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is closed but is not open")
        if len(set(slots)) != len(slots):
            raise CacheError(f"a slot is closed twice in one call: {slots}")
        for s in slots:
            for g in self._groups:
                g.pool.give_back(g.pages.pop(s))
            self.lengths[s] = 0
        self.slots.give_back(slots)

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        return self.lengths[slot]

    def free_pages(self) -> list[int]:
        return [g.pool.n_free for g in self._groups]

    # ------------------------------------------------------------------ growing
    def reserve(self, wants: dict) -> None:
        """Make room for each slot to hold ``wants[slot]`` tokens, or change nothing and raise."""
        need = [0] * len(self._groups)
        for slot, n_tokens in wants.items():
            if not self.slots.is_held(slot):
                raise CacheError(f"slot {slot} is not open")
            if n_tokens > self.max_seq_len:
                raise CacheFull(f"slot {slot} would hold {n_tokens} tokens; the longest sequence allowed "
                                f"is {self.max_seq_len}")
            for gi, g in enumerate(self._groups):
                need[gi] += max(0, pages_for(n_tokens) - len(g.pages[slot]))
        for gi, g in enumerate(self._groups):
            if need[gi] > g.pool.n_free:
                raise CacheFull(f"{need[gi]} more pages wanted, {g.pool.n_free} of {g.pool.n} free "
                                f"(max_tokens={self.max_tokens})")
        for slot, n_tokens in wants.items():
            for g in self._groups:
                more = pages_for(n_tokens) - len(g.pages[slot])
                if more > 0:
                    g.pages[slot].extend(g.pool.take(more))

    def advance(self, slot: int, n_new: int) -> None:
        self.lengths[slot] += n_new

    def truncate(self, slot: int, length: int) -> None:
        """Forget the tokens from ``length`` on (the reference's rewind for attention-only models,
        core/runtime.cpp:2804-2811).  Not possible once a mixer keeps fixed-size state."""
        if self._unit_state:
            raise CacheError("a sequence with fixed-size state cannot be truncated")
        if not 0 <= length <= self.length(slot):
            raise CacheError(f"slot {slot} holds {self.lengths[slot]} tokens, cannot truncate to {length}")
        self.lengths[slot] = length
        for g in self._groups:
            keep = pages_for(length)
            g.pool.give_back(g.pages[slot][keep:])
            del g.pages[slot][keep:]

    # ------------------------------------------------------------------ page tables
    def page_table_host(self, gid: int, slots) -> np.ndarray:
        """[len(slots), table_width] int32; entries beyond a sequence's pages are 0 and never read."""
        g = self._groups[gid]
        table = np.zeros((len(slots), self.table_width), dtype=np.int32)
        for r, s in enumerate(slots):
            p = g.pages[s]
            table[r, :len(p)] = p
        return table
