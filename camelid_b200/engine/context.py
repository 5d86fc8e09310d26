"""What a step looks like to the parts: the packed rows of a batch and where they belong.

All sequences of a step are packed row after row: sequence ``i`` owns rows
``seq_row0[i] .. seq_row0[i] + seq_new[i]``; row ``r`` has token ``tokens[r]``, belongs to
sequence ``row_seq[r]`` and sits at absolute position ``row_pos[r]`` (the sequence's
length before the step plus its offset). There is no padding, so there is nothing that
padding could change. The integer arrays reach the device in one copy.
"""
from __future__ import annotations

import torch

from ..cache.book import PAGE


class Workspace:
    """Named device buffers that live from step to step and only ever grow."""

    def __init__(self, device):
        self.device = device
        self._bufs: dict = {}

    def get(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:n].view(shape)


class StepContext:
    def __init__(self, *, cache, workspace: Workspace, dtype: torch.dtype, device, slots: list, starts: list,
                 tokens: list, want: list):
        self.cache = cache
        self.ws = workspace
        self.dtype = dtype
        self.device = device
        self.h_slots = list(slots)
        self.h_start = list(starts)
        self.h_new = [len(t) for t in tokens]
        self.n_seqs = len(slots)
        self.n_rows = sum(self.h_new)
        self.max_new = max(self.h_new)
        self.max_len = max(s + n for s, n in zip(self.h_start, self.h_new))
        self.decode = self.max_new == 1
        self.entry = -1                 # schedule entry that is running
        self.cache_source = None        # entry whose keys and values the running entry reads
        row0, acc = [], 0
        for n in self.h_new:
            row0.append(acc)
            acc += n
        self.h_row0 = row0
        want_rows = [row0[i] + w for i, ws in enumerate(want) for w in ws]
        self.n_want = len(want_rows)
        flat_tokens = [t for ts in tokens for t in ts]
        row_seq = [i for i, n in enumerate(self.h_new) for _ in range(n)]
        row_pos = [self.h_start[i] + j for i, n in enumerate(self.h_new) for j in range(n)]
        n_groups = len(cache.book.kv_specs) if cache is not None else 0
        tables = [cache.book.block_table(g, self.h_slots) for g in range(n_groups)]
        self._table_width = [len(t[0]) for t in tables]
        parts = [flat_tokens, row_seq, row_pos, self.h_slots, self.h_start, self.h_new, row0, want_rows]
        for t in tables:
            parts.append([p for row in t for p in row])
        sizes = [len(p) for p in parts]
        host = torch.tensor([x for p in parts for x in p], dtype=torch.int32)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        dev = host.to(device, non_blocking=True)
        self._host_meta = host            # keep the pinned buffer alive until the copy ran
        views, off = [], 0
        for n in sizes:
            views.append(dev[off:off + n])
            off += n
        (self.tokens, self.row_seq, self.row_pos, self.seq_slot, self.seq_start, self.seq_new, self.seq_row0,
         self.want_rows) = views[:8]
        self._tables = [views[8 + g].view(self.n_seqs, self._table_width[g]) for g in range(n_groups)]
        self._tiles: dict = {}
        self.h2d_bytes = host.numel() * 4

    # ---- helpers for parts ----
    def buffer(self, name: str, shape: tuple, dtype: torch.dtype | None = None) -> torch.Tensor:
        return self.ws.get(name, shape, dtype or self.dtype)

    def block_table(self, group: int) -> torch.Tensor:
        """int32 [sequences, blocks]: page of each block of each sequence of the step."""
        return self._tables[group]

    def kv(self):
        """(group, key pages, value pages) the running entry reads and, unless it borrows
        them from another entry, writes."""
        entry = self.cache_source if self.cache_source is not None else self.entry
        return self.cache.kv_pages(entry)

    def state(self) -> torch.Tensor:
        """[slots, *shape] fixed-size state of the running entry; index it with ``seq_slot``."""
        return self.cache.state_of(self.entry)

    def query_tiles(self, rows_per_tile: int):
        """Tiles of at most ``rows_per_tile`` consecutive new rows of one sequence:
        (tile_seq, tile_q0, n_tiles) on the device."""
        got = self._tiles.get(rows_per_tile)
        if got is None:
            seqs, q0s = [], []
            for i, n in enumerate(self.h_new):
                for q0 in range(0, n, rows_per_tile):
                    seqs.append(i)
                    q0s.append(q0)
            t = torch.tensor(seqs + q0s, dtype=torch.int32)
            if torch.device(self.device).type == "cuda":
                t = t.pin_memory()
            d = t.to(self.device, non_blocking=True)
            got = (d[:len(seqs)], d[len(seqs):], len(seqs), t)
            self._tiles[rows_per_tile] = got
            self.h2d_bytes += t.numel() * 4
        return got[0], got[1], got[2]

    @property
    def max_blocks_in_use(self) -> int:
        return (self.max_len + PAGE - 1) // PAGE
