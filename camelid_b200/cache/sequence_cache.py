"""The cache on the device: page pools for keys and values, and fixed-size state per slot.

Each schedule entry of the model states what its mixer needs (a ``KVSpec``, a
``StateSpec`` or nothing). Entries with equal ``KVSpec`` share one group: one tensor
``[entries, pages, kv_heads, 64, head_dim]`` for keys and one for values, in the compute
type, and one page pool. Entries with equal ``StateSpec`` share one tensor
``[entries, slots, *shape]``. An entry that reads another entry's cache has no storage.
The dense Llama decoder has one group (all keys, every layer) and no state.

The reference's device cache is ``cache_k/cache_v`` as ``[kv_head][position][head_dim]``
per layer (src/cuda_resident.rs:5424-5428, :1568-1583), sized from the configuration and
refused before allocation when it does not fit (src/inference/kv_cache.rs:285-299).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..errors import CacheError
from .book import PAGE, CacheBook, KVSpec, StateSpec

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class SequenceCache:
    def __init__(self, entry_specs: list, entry_sources: list, *, max_tokens: int, max_position: int,
                 dtype: torch.dtype, device, max_slots: Optional[int] = None):
        n_pages = max(1, (int(max_tokens) + PAGE - 1) // PAGE)
        n_slots = int(max_slots) if max_slots else n_pages
        self.dtype = dtype
        self.device = torch.device(device)
        self.entry_specs = list(entry_specs)
        self.entry_sources = list(entry_sources)
        kv_specs: list = []
        state_specs: list = []
        self.entry_kv: list = [None] * len(entry_specs)        # (group, index in group)
        self.entry_state: list = [None] * len(entry_specs)
        counts_kv: list = []
        counts_state: list = []
        for i, (spec, src) in enumerate(zip(entry_specs, entry_sources)):
            if src is not None:
                continue
            if isinstance(spec, KVSpec):
                if spec not in kv_specs:
                    kv_specs.append(spec)
                    counts_kv.append(0)
                g = kv_specs.index(spec)
                self.entry_kv[i] = (g, counts_kv[g])
                counts_kv[g] += 1
            elif isinstance(spec, StateSpec):
                if spec not in state_specs:
                    state_specs.append(spec)
                    counts_state.append(0)
                g = state_specs.index(spec)
                self.entry_state[i] = (g, counts_state[g])
                counts_state[g] += 1
            elif spec is not None:
                raise CacheError(f"schedule entry {i}: unknown cache need {spec!r}")
        for i, src in enumerate(entry_sources):
            if src is not None:
                if self.entry_kv[src] is None:
                    raise CacheError(f"schedule entry {i} reads the keys of entry {src}, which keeps none")
                self.entry_kv[i] = self.entry_kv[src]
        self.book = CacheBook(kv_specs, n_pages, n_slots, max_position)
        need = self.bytes_needed(kv_specs, counts_kv, state_specs, counts_state, n_pages, n_slots, dtype)
        if self.device.type == "cuda":
            free, _total = torch.cuda.mem_get_info(self.device)
            if need > free:
                raise CacheError(f"the cache needs {need} bytes ({n_pages} pages of {PAGE} tokens) but only {free} are free on {self.device}")
        # zero-filled once; kernels never count rows beyond a sequence's length
        self.k = [torch.zeros((counts_kv[g], n_pages, s.n_kv_heads, PAGE, s.head_dim), dtype=dtype, device=self.device)
                  for g, s in enumerate(kv_specs)]
        self.v = [torch.zeros_like(t) for t in self.k]
        self.state = [torch.zeros((counts_state[g], n_slots) + tuple(s.shape), dtype=_STATE_DTYPES[s.dtype],
                                  device=self.device) for g, s in enumerate(state_specs)]
        self.bytes = need

    @staticmethod
    def bytes_needed(kv_specs, counts_kv, state_specs, counts_state, n_pages, n_slots, dtype) -> int:
        size = torch.empty((), dtype=dtype).element_size()
        total = 0
        for s, c in zip(kv_specs, counts_kv):
            total += 2 * c * n_pages * s.n_kv_heads * PAGE * s.head_dim * size
        for s, c in zip(state_specs, counts_state):
            n = 1
            for d in s.shape:
                n *= d
            total += c * n_slots * n * torch.empty((), dtype=_STATE_DTYPES[s.dtype]).element_size()
        return total

    # ---- slots ----
    def alloc_slot(self) -> int:
        slot = self.book.alloc_slot()
        for t in self.state:
            t[:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        self.book.free_slot(slot)

    def length(self, slot: int) -> int:
        self.book._check_slot(slot)
        return self.book.length[slot]

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions of ``slot`` at and beyond ``length`` (the reference's
        ``rollback_to_position``, src/inference/kv_cache.rs:246-269). State of fixed size has no
        positions to go back to: a cache that keeps any refuses."""
        if self.state and length < self.length(slot):
            raise CacheError(f"slot {slot}: this model keeps per-sequence state of fixed size, which cannot be rolled back")
        self.book.truncate(slot, length)

    # ---- storage of one schedule entry ----
    def kv_pages(self, entry: int):
        """(group, keys [pages, kv_heads, 64, head_dim], values) of a schedule entry."""
        where = self.entry_kv[entry]
        if where is None:
            raise CacheError(f"schedule entry {entry} keeps no keys and values")
        g, i = where
        return g, self.k[g][i], self.v[g][i]

    def state_of(self, entry: int) -> torch.Tensor:
        """[slots, *shape] state of a schedule entry."""
        where = self.entry_state[entry]
        if where is None:
            raise CacheError(f"schedule entry {entry} keeps no per-sequence state")
        g, i = where
        return self.state[g][i]
