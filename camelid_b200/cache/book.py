"""Bookkeeping of the cache, without any device memory: slots, pages and lengths.

A *slot* stands for one live sequence. A *page* holds the keys and values of 64
consecutive positions of one sequence (for every layer entry of its group). Layer entries
whose mixers ask for the same kind of storage form a *group* with a page pool of its own;
a group with a window gives pages back as soon as no later query can see them. Slots and
pages are handed out lowest id first and are used again after they are freed.

The reference keeps one history per engine (src/cuda_resident.rs:5424-5428) with a cursor
and a rollback (src/inference/kv_cache.rs:246-269) and refuses an append past the context
before any write (src/inference.rs:4106-4111, src/inference/kv_cache.rs:275-280); slots,
pages and groups are this library's own.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass
from typing import Optional

from ..errors import CacheError

PAGE = 64


@dataclass(frozen=True)
class KVSpec:
    """Keys and values per position: ``window`` None keeps all of them, an integer keeps the
    last ``window`` positions."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per sequence: a tensor of ``shape`` and ``dtype`` for every slot,
    zeroed when the slot is handed out."""
    shape: tuple
    dtype: str = "float32"


class FreeList:
    """Ids 0..n-1; the lowest free id is handed out first."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n))
        heapq.heapify(self._free)
        self._held = [False] * n

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} (all {self.n} are in use)")
        i = heapq.heappop(self._free)
        self._held[i] = True
        return i

    def free(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is not in use (freed twice?)")
        self._held[i] = False
        heapq.heappush(self._free, i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)


class CacheBook:
    """Who holds what. ``kv_specs`` lists the distinct KVSpec of the model, one page pool each."""

    def __init__(self, kv_specs: list, n_pages: int, n_slots: int, max_position: int):
        if n_pages < 1 or n_slots < 1:
            raise CacheError(f"a cache needs at least one page and one slot (got {n_pages} pages, {n_slots} slots)")
        self.kv_specs = list(kv_specs)
        self.n_pages = n_pages
        self.n_slots = n_slots
        self.max_position = max_position
        self.slots = FreeList(n_slots, "slot")
        self.pools = [FreeList(n_pages, f"page of group {g}") for g in range(len(self.kv_specs))]
        self.length = [0] * n_slots
        # pages[group][slot] : list of page ids by block index; -1 where a windowed group gave one back
        self.pages = [[[] for _ in range(n_slots)] for _ in self.kv_specs]
        self.generation = [0] * n_slots        # bumped whenever a slot's pages change

    # ---- slots ----
    def alloc_slot(self) -> int:
        s = self.slots.alloc()
        self.length[s] = 0
        return s

    def free_slot(self, slot: int) -> None:
        self._check_slot(slot)
        for g, pool in enumerate(self.pools):
            for p in self.pages[g][slot]:
                if p >= 0:
                    pool.free(p)
            self.pages[g][slot] = []
        self.length[slot] = 0
        self.generation[slot] += 1
        self.slots.free(slot)

    def _check_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not in use")

    # ---- pages ----
    def _first_needed_block(self, g: int, length_before: int) -> int:
        """First block a query at a position >= length_before can still see."""
        w = self.kv_specs[g].window
        if w is None:
            return 0
        return max(0, length_before - w + 1) // PAGE

    def pages_needed(self, slot: int, new_length: int) -> list:
        """Pages each group has to add so that positions < new_length have storage."""
        need_blocks = (new_length + PAGE - 1) // PAGE
        return [max(0, need_blocks - len(self.pages[g][slot])) for g in range(len(self.pools))]

    def check_extend(self, requests: list) -> None:
        """``requests``: (slot, tokens to add). Raises before anything changes if a slot is
        unknown or occurs twice, a sequence would pass the model's maximum position, or a
        pool has too few free pages for all requests together."""
        seen = set()
        want = [0] * len(self.pools)
        for slot, n_new in requests:
            self._check_slot(slot)
            if slot in seen:
                raise CacheError(f"slot {slot} occurs twice in one step")
            seen.add(slot)
            if n_new < 1:
                raise CacheError(f"slot {slot}: a step must bring at least one token")
            new_len = self.length[slot] + n_new
            if new_len > self.max_position:
                raise CacheError(f"slot {slot}: {new_len} positions exceed the model's maximum of {self.max_position}")
            for g, n in enumerate(self.pages_needed(slot, new_len)):
                want[g] += n
        for g, pool in enumerate(self.pools):
            if want[g] > pool.n_free:
                raise CacheError(f"cache is full: group {g} needs {want[g]} more pages, {pool.n_free} of {pool.n} are free")

    def extend(self, slot: int, n_new: int) -> int:
        """Give ``slot`` storage for ``n_new`` more positions (call check_extend first);
        returns the length before. The length itself moves with ``commit``."""
        start = self.length[slot]
        changed = False
        for g, n in enumerate(self.pages_needed(slot, start + n_new)):
            for _ in range(n):
                self.pages[g][slot].append(self.pools[g].alloc())
                changed = True
        if changed:
            self.generation[slot] += 1
        return start

    def commit(self, slot: int, n_new: int) -> None:
        """The step ran: the sequence is n_new longer; windowed groups give back the pages
        that no later query can see."""
        self.length[slot] += n_new
        for g in range(len(self.pools)):
            first = self._first_needed_block(g, self.length[slot])
            pages = self.pages[g][slot]
            for b in range(min(first, len(pages))):
                if pages[b] >= 0:
                    self.pools[g].free(pages[b])
                    pages[b] = -1
                    self.generation[slot] += 1

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions at and beyond ``length`` (the reference's rollback)."""
        self._check_slot(slot)
        if not 0 <= length <= self.length[slot]:
            raise CacheError(f"slot {slot}: cannot truncate from {self.length[slot]} to {length}")
        for g in range(len(self.pools)):
            if self.kv_specs[g].window is not None and length < self.length[slot]:
                first = self._first_needed_block(g, length)
                if any(p < 0 for p in self.pages[g][slot][first:(length + PAGE - 1) // PAGE]):
                    raise CacheError(f"slot {slot}: group {g} has already given back positions before {length}")
            keep = (length + PAGE - 1) // PAGE
            pages = self.pages[g][slot]
            while len(pages) > keep:
                p = pages.pop()
                if p >= 0:
                    self.pools[g].free(p)
        self.length[slot] = length
        self.generation[slot] += 1

    def block_table(self, g: int, slots: list, width: int | None = None) -> list:
        """Rows of page ids by block index for the given slots, padded with -1 to one width."""
        rows = [self.pages[g][s] for s in slots]
        width = max([width or 1] + [len(r) for r in rows])
        return [r + [-1] * (width - len(r)) for r in rows]

    def audit(self) -> None:
        """Every page is free or held by exactly one slot; every held slot is known."""
        for g, pool in enumerate(self.pools):
            held = [p for s in range(self.n_slots) for p in self.pages[g][s] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page is held twice")
            if len(held) != pool.n_held:
                raise CacheError(f"group {g}: {pool.n_held} pages are out but slots hold {len(held)}")
            for s in range(self.n_slots):
                if self.pages[g][s] and not self.slots.is_held(s):
                    raise CacheError(f"group {g}: free slot {s} still holds pages")
