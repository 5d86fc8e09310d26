"""What a step looks like to the parts: the packed rows of a batch and where they belong.

All sequences of a step are packed row after row: sequence ``i`` owns rows
``seq_row0[i] .. seq_row0[i] + seq_new[i]``; row ``r`` has token ``tokens[r]``, belongs to
sequence ``row_seq[r]`` and sits at absolute position ``row_pos[r]`` (the sequence's
length before the step plus its offset). There is no padding, so there is nothing that
padding could change. All integer arrays of a step lie in one buffer and reach the device
in one copy; a decode step of a fixed batch size always has the same layout, which is what
lets it run as a captured CUDA graph on a static buffer.
"""
from __future__ import annotations

import weakref

import numpy as np
import torch

from ..cache.book import PAGE
from ..csrc import ops
from ..errors import KernelError
from ..options import KernelOptions


class Workspace:
    """Named device buffers that live from step to step and only ever grow."""

    def __init__(self, device):
        self.device = device
        self._bufs: dict = {}
        self._views: dict = {}          # (name, dtype, shape) -> view: steps of a size seen before make no new tensors

    def get(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(shape)
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self._views = {k: v for k, v in self._views.items() if k[:2] != key}
        if len(self._views) > 4096:
            self._views.clear()
        view = buf[:n].view(shape)
        self._views[(name, dtype, shape)] = view
        return view


class StepLayout:
    """Offsets of a step's integer arrays in its one buffer: tokens first (so that a decode
    loop that keeps its tokens on the device can copy everything but them), then rows,
    sequences, wanted rows, one block table per cache group, and the query tiles."""

    def __init__(self, n_rows: int, n_seqs: int, n_want: int, table_widths: list, n_tiles: dict):
        self.n_rows, self.n_seqs, self.n_want = n_rows, n_seqs, n_want
        self.n_tiles = dict(n_tiles)                   # rows per tile -> number of tiles
        self.table_widths = list(table_widths)
        names = [("tokens", n_rows), ("row_seq", n_rows), ("row_pos", n_rows), ("seq_slot", n_seqs),
                 ("seq_start", n_seqs), ("seq_new", n_seqs), ("seq_row0", n_seqs), ("want_rows", n_want)]
        names += [(f"table{g}", n_seqs * w) for g, w in enumerate(table_widths)]
        for r, n in self.n_tiles.items():
            names += [(f"tile_seq{r}", n), (f"tile_q0{r}", n)]
        self.offsets, off = {}, 0
        for name, n in names:
            self.offsets[name] = (off, n)
            off += n
        self.total = off

    def view(self, buf, name):
        off, n = self.offsets[name]
        return buf[off:off + n]


class StepContext:
    """Built per step by the engine (``for_step``) or once for a captured decode graph
    (``static``); parts read it and never change it."""

    # ---- construction ----
    def __init__(self, *, cache, workspace: Workspace, dtype: torch.dtype, device, layout: StepLayout,
                 meta_dev: torch.Tensor, options: KernelOptions | None = None):
        # the context of a captured graph lives as long as the graph: it must not keep the cache alive
        self._cache = weakref.ref(cache) if cache is not None else None
        self.options = options if options is not None else KernelOptions()
        self.ws = workspace
        self.dtype = dtype
        self.device = device
        self.layout = layout
        self.meta_dev = meta_dev
        self.n_rows, self.n_seqs, self.n_want = layout.n_rows, layout.n_seqs, layout.n_want
        v = lambda name: layout.view(meta_dev, name)        # noqa: E731
        self.tokens, self.row_seq, self.row_pos = v("tokens"), v("row_seq"), v("row_pos")
        self.seq_slot, self.seq_start, self.seq_new = v("seq_slot"), v("seq_start"), v("seq_new")
        self.seq_row0, self.want_rows = v("seq_row0"), v("want_rows")
        self._tables = [v(f"table{g}").view(layout.n_seqs, w) for g, w in enumerate(layout.table_widths)]
        self._tiles = {r: (v(f"tile_seq{r}"), v(f"tile_q0{r}"), n) for r, n in layout.n_tiles.items()}
        self.entry = -1                 # schedule entry that is running
        self.cache_source = None        # entry whose keys and values the running entry reads
        self.pending = None             # float32 [splits, rows, hidden] still to be added to the residual stream
        self.deferred = None            # (x, w, residual): a product into the residual stream not yet launched
        self.row_scale = None           # ops.RowScale: what the rows of the last norm's output still lack
        # host-side knowledge (filled by the constructors below)
        self.h_slots: list = []
        self.h_start: list = []
        self.h_new: list = []
        self.h_row0: list = []
        self.max_new = 1
        self.max_len = 1
        self.decode = True
        self.h2d_bytes = 0

    @property
    def cache(self):
        return self._cache() if self._cache is not None else None

    @staticmethod
    def host_arrays(slots, starts, tokens, want, tables, tile_sizes):
        """The step's integer arrays as one int32 numpy vector, with its layout. ``tokens``: one
        list or integer array per sequence."""
        tokens = [np.asarray(t).reshape(-1) for t in tokens]
        news = [int(t.size) for t in tokens]
        row0 = np.zeros(len(news), dtype=np.int64)
        if len(news) > 1:
            row0[1:] = np.cumsum(news[:-1])
        n_rows = int(sum(news))
        flat = np.concatenate(tokens).astype(np.int32, copy=False)
        row_seq = np.repeat(np.arange(len(news), dtype=np.int32), news)
        row_pos = (np.arange(n_rows, dtype=np.int64) - np.repeat(row0, news) + np.repeat(np.asarray(starts), news))
        want_rows = [int(row0[i]) + w for i, ws in enumerate(want) for w in ws]
        tiles = {}
        for r in (tile_sizes if max(news) > 1 else [1]):
            tile_seq, tile_q0 = [], []
            for i, n in enumerate(news):
                q0s = range(0, n, r)
                tile_seq += [i] * len(q0s)
                tile_q0 += q0s
            tiles[r] = (tile_seq, tile_q0)
        layout = StepLayout(n_rows, len(news), len(want_rows), [len(t[0]) for t in tables],
                            {r: len(t[0]) for r, t in tiles.items()})
        parts = [flat, row_seq, row_pos.astype(np.int32), np.asarray(slots, dtype=np.int32),
                 np.asarray(starts, dtype=np.int32), np.asarray(news, dtype=np.int32), row0.astype(np.int32),
                 np.asarray(want_rows, dtype=np.int32)]
        parts += [np.asarray(t, dtype=np.int32).reshape(-1) for t in tables]
        for tile_seq, tile_q0 in tiles.values():
            parts += [np.asarray(tile_seq, dtype=np.int32), np.asarray(tile_q0, dtype=np.int32)]
        return layout, np.concatenate(parts), news, row0.tolist()

    @classmethod
    def for_step(cls, *, cache, workspace, dtype, device, slots, starts, tokens, want, tile_sizes=(1,), options=None):
        """A context for one eager step: arrays built on the host and sent in one copy."""
        n_groups = len(cache.book.kv_specs) if cache is not None else 0
        tables = [cache.book.block_table(g, list(slots)) for g in range(n_groups)]
        layout, host, news, row0 = cls.host_arrays(slots, starts, tokens, want, tables, list(tile_sizes))
        t = torch.from_numpy(host)
        if torch.device(device).type == "cuda":
            t = t.pin_memory()
        ctx = cls(cache=cache, workspace=workspace, dtype=dtype, device=device, layout=layout,
                  meta_dev=t.to(device, non_blocking=True), options=options)
        ctx._host_meta = t                # keep the pinned buffer alive until the copy ran
        ctx._set_host(slots, starts, news, row0)
        ctx.h2d_bytes = host.nbytes
        return ctx

    @classmethod
    def static(cls, *, cache, workspace, dtype, device, n_seqs, table_widths, options=None):
        """A context on a fixed buffer for decode steps of ``n_seqs`` sequences (one token each,
        every sequence's logits wanted); ``meta_dev`` is refilled before every replay."""
        layout = StepLayout(n_seqs, n_seqs, n_seqs, table_widths, {1: n_seqs})
        meta = torch.zeros(layout.total, dtype=torch.int32, device=device)
        ctx = cls(cache=cache, workspace=workspace, dtype=dtype, device=device, layout=layout, meta_dev=meta,
                  options=options)
        ctx._set_host([0] * n_seqs, [0] * n_seqs, [1] * n_seqs, list(range(n_seqs)))
        ctx.max_len = max(table_widths) * PAGE if table_widths else 1
        return ctx

    def _set_host(self, slots, starts, news, row0):
        self.h_slots, self.h_start, self.h_new, self.h_row0 = list(slots), list(starts), list(news), list(row0)
        self.max_new = max(news)
        self.max_len = max(s + n for s, n in zip(starts, news))
        self.decode = self.max_new == 1

    # ---- helpers for parts ----
    def settle(self, residual: torch.Tensor) -> None:
        """Add what is pending to the residual stream now. A norm that reads the stream next does
        this itself in its own kernel; parts that touch the stream otherwise call this first."""
        if self.deferred is not None:
            from ..parts import linear
            linear.run_deferred(self)
        if self.pending is not None:
            part, self.pending = self.pending, None
            ops.add_partials(residual, part)

    def take_row_scale(self):
        """The scale the rows of the last norm's output still lack (None if they are complete).
        Whoever takes it applies it: a product may scale its own output rows instead."""
        scale, self.row_scale = self.row_scale, None
        return scale

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
        if self.decode:                       # one row per sequence: every tiling is the same
            return self._tiles[1]
        try:
            return self._tiles[rows_per_tile]
        except KeyError:
            raise KernelError(f"this step has tiles of {sorted(self._tiles)} rows, not of {rows_per_tile}; the "
                             f"mixer's query_tile_sizes() must name every size it uses") from None

    @property
    def max_blocks_in_use(self) -> int:
        return (self.max_len + PAGE - 1) // PAGE
