"""Decode steps as captured CUDA graphs.

A decode step of a fixed number of sequences always launches the same kernels on the same
buffers; only the integer arrays of the step change. So the step is captured once per
(batch size, block-table widths) on a static context and replayed: per step the host fills
a pinned copy of the arrays, sends it in one copy, and launches the graph. With ``feed`` the
graph also picks the next token greedily and writes it where the next step reads its
tokens, so a decode loop can run without any traffic to the host.

The reference measured CUDA graphs as a loss on its 7.9 ms/token regime
(src/cuda_resident.rs:5558-5571); at a few hundred microseconds per step on a B200 the
launch gaps are most of the step without them.
"""
from __future__ import annotations

import weakref

import numpy as np
import torch

from ..csrc import ops
from .context import StepContext, Workspace

_RING = 4


def bucket_width(blocks: int) -> int:
    """Block-table width a graph is captured for: the next power of two, at least 4."""
    w = 4
    while w < blocks:
        w *= 2
    return w


class DecodeGraph:
    def __init__(self, model, cache, n_seqs: int, widths: list, feed: bool, adjust: bool = False):
        self.model, self.n_seqs, self.widths, self.feed, self.adjust = model, n_seqs, list(widths), feed, adjust
        self._cache = weakref.ref(cache)        # the model keeps its graphs per cache and drops them with it
        dev = model.device
        self.ctx = StepContext.static(cache=cache, workspace=Workspace(dev), dtype=model.dtype, device=dev,
                                      n_seqs=n_seqs, table_widths=self.widths, options=model.options)
        lay = self.ctx.layout
        self.host = [torch.zeros(lay.total, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.host_np = [h.numpy() for h in self.host]
        self.events = [None] * _RING
        self.turn = 0
        ar = np.arange(n_seqs, dtype=np.int32)
        for h in self.host_np:
            for name, val in (("row_seq", ar), ("seq_new", 1), ("seq_row0", ar), ("want_rows", ar), ("tile_seq1", ar),
                              ("tile_q01", 0)):
                lay.view(h, name)[:] = val
        self.graph = None
        self.logits = None
        self.next_tokens = None
        self.launches = 0
        self._table_key = [None] * _RING
        if feed and feed is not True:              # a sampling step: seed, temperature and filters live on the device,
            self.seed = torch.zeros(1, dtype=torch.int64, device=dev)          # so one graph replays for any of them
            self.draws = torch.zeros(n_seqs, dtype=torch.float32, device=dev)
            self.sample_params = torch.tensor([1.0, 0.0, 1.0, 0.0], dtype=torch.float32, device=dev)
        if adjust:
            # Bias and penalties inside a step that feeds itself: how often each token stands in a row's
            # history is kept on the device (set from the histories when a run starts, the chosen tokens
            # counted by the step), the bias as a dense row, the three penalties as numbers in device memory.
            assert feed, "adjustments on the device belong to steps that pick their own token"
            self.counts = torch.zeros(n_seqs, model.vocab_size, dtype=torch.int32, device=dev)
            self.bias = torch.zeros(model.vocab_size, dtype=torch.float32, device=dev)
            self.penalties = torch.zeros(3, dtype=torch.float32, device=dev)
            self.counts_host = torch.zeros(n_seqs, model.vocab_size, dtype=torch.int32).pin_memory()

    @property
    def cache(self):
        return self._cache()

    def fill(self, slots: list, starts: list, tokens) -> int:
        """Write the step's arrays into the next pinned buffer; returns its index."""
        i = self.turn
        self.turn = (self.turn + 1) % _RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        lay, h = self.ctx.layout, self.host_np[i]
        if tokens is not None:
            lay.view(h, "tokens")[:] = tokens
        lay.view(h, "row_pos")[:] = starts
        lay.view(h, "seq_start")[:] = starts
        lay.view(h, "seq_slot")[:] = slots
        book = self.cache.book
        key = tuple((s, book.generation[s]) for s in slots)
        if self._table_key[i] != key:
            for g, w in enumerate(self.widths):
                lay.view(h, f"table{g}")[:] = np.asarray(book.block_table(g, slots, width=w), dtype=np.int32).reshape(-1)
            self._table_key[i] = key
        return i

    def send(self, i: int, with_tokens: bool) -> int:
        """One copy of the arrays to the device (without the tokens when the device has them)."""
        skip = 0 if with_tokens else self.n_seqs
        self.ctx.meta_dev[skip:].copy_(self.host[i][skip:], non_blocking=True)
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return (self.ctx.layout.total - skip) * 4

    def _forward(self):
        logits = self.model.run(self.ctx)
        if self.adjust:
            ops.adjust_dense(logits, self.counts, self.bias, self.penalties)
        if self.feed is True:
            ops.argmax_rows(logits, self.ctx.tokens, self.model.logit_error_word())
        elif self.feed:          # "sample": the draw from the seed and the position, the rest from sample_params
            ops.draws_at(self.ctx.row_pos, self.seed, self.draws)
            ops.sample_rows(logits, 1.0, 0, 1.0, 0.0, self.draws, self.ctx.tokens, self.model.logit_error_word(),
                            params=self.sample_params)
        if self.adjust:
            ops.count_tokens(self.ctx.tokens, self.counts)
        return logits

    def capture(self):
        """Warm up eagerly on the buffer's present contents, then capture. The warm-up runs the
        step once for real: keys and values it writes are written again, identically, by the
        first replay, but per-sequence state of fixed size would be advanced twice, so it is put
        back as it was."""
        tokens_before = self.ctx.tokens.clone()
        state_before = [t.clone() for t in self.cache.state]
        self._forward()
        self.ctx.tokens.copy_(tokens_before)
        for t, saved in zip(self.cache.state, state_before):
            t.copy_(saved)
        torch.cuda.synchronize()
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.logits = self._forward()
        self.launches = ops.launch_count() - before
        self.graph = g

    def replay(self):
        self.graph.replay()
        ops.add_launches(self.launches)
        return self.logits

    def native_loop(self, err: torch.Tensor):
        """The C++ decode loop bound to this graph (made at its first use, after capture).
        ``err``: the sampler's error word (non-finite logits)."""
        if getattr(self, "_native", None) is None or self._native.err is not err:
            self._native = ops.NativeDecodeLoop(self.n_seqs, self.ctx.layout, self.ctx.meta_dev, self.host_np[0],
                                                self.logits, err)
        return self._native

    def run_native(self, slots: list, starts: list, tokens: list, history_lens: list, max_steps: int, stop_ids,
                   temperature: float, top_k, top_p, min_p, seed, err: torch.Tensor):
        """Up to ``max_steps`` steps in C++ (the cache must already hold pages for them). Returns
        (tokens [steps, sequences] as a numpy array, steps done)."""
        i = self.fill(slots, starts, tokens)
        self.send(i, with_tokens=True)                  # block tables and the static arrays
        if self.graph is None:
            self.capture()
        loop = self.native_loop(err)
        return loop.run(self.graph.raw_cuda_graph_exec(), tokens, starts, slots, history_lens, max_steps, stop_ids,
                        temperature, top_k, top_p, min_p, seed, self.launches)

    def run_fed(self, slots: list, starts: list, tokens: list, steps: int, seed: int = 0, histories=None, options=None):
        """``steps`` steps of a graph captured with ``feed`` (greedy, or sampling with the draws
        made on the device from ``seed`` and each row's position), queued at once by the C++
        loop: the device feeds itself, the host sends positions and reads the chosen tokens.
        A graph with adjustments needs ``histories`` (per sequence the tokens so far, the one fed
        first included) and ``options`` (the penalties and the bias). Returns the tokens
        [steps, sequences] as a numpy array."""
        assert self.feed
        if self.feed is not True:
            signed = int(seed) & ((1 << 64) - 1)
            self.seed.fill_(signed - (1 << 64) if signed >= (1 << 63) else signed)
            now = (float(options.temperature), float(options.top_k or 0),
                   float(options.top_p if options.top_p is not None else 1.0), float(options.min_p or 0.0))
            if now != getattr(self, "_sample_now", None):
                self.sample_params.copy_(torch.tensor(now, dtype=torch.float32))
                self._sample_now = now
        i = self.fill(slots, starts, tokens)
        self.send(i, with_tokens=True)                  # block tables and the static arrays
        if self.graph is None:
            self.capture()
        if self.adjust:
            # What the device holds after a run is what the next run of the same sequences starts from: the
            # histories' counts are sent again only if this is not that next run (same slots in the same use,
            # histories grown by exactly the run's steps, the run's last tokens fed, the same options).
            book = self.cache.book
            now = (tuple((s, book.generation[s]) for s in slots), tuple(len(h) for h in histories),
                   tuple(int(t) for t in tokens), self._options_key(options))
            if now != getattr(self, "_adjust_next", None):
                self._set_adjustments(histories, options)
        if getattr(self, "_fed", None) is None:
            self._fed = ops.FedDecodeLoop(self.n_seqs, self.ctx.layout, self.ctx.meta_dev, self.host_np[i])
        out = []
        done = 0
        while done < steps:
            k = min(steps - done, self._fed.RING)
            first = tokens if done == 0 else out[-1][-1]
            out.append(self._fed.run(self.graph.raw_cuda_graph_exec(), first, [s + done for s in starts], slots, k,
                                     self.launches))
            done += k
        result = np.concatenate(out) if len(out) > 1 else out[0]
        if self.adjust:
            book = self.cache.book
            self._adjust_next = (tuple((s, book.generation[s]) for s in slots), tuple(len(h) + steps for h in histories),
                                 tuple(int(t) for t in result[-1]), self._options_key(options))
        return result


    @staticmethod
    def _options_key(options) -> tuple:
        return (options.repeat_penalty, options.presence_penalty, options.frequency_penalty,
                tuple((int(t), float(b)) for t, b in options.logit_bias))

    def _set_adjustments(self, histories, options) -> None:
        """Counts of each row's history, the dense bias and the penalties to the device (after the
        capture, whose warm-up step counted a token of its own)."""
        vocab = self.model.vocab_size
        host = self.counts_host.numpy()
        penalise = options.presence_penalty != 0.0 or options.frequency_penalty != 0.0 or options.repeat_penalty != 1.0
        for r, hist in enumerate(histories):
            if penalise:
                h = np.asarray(hist, dtype=np.int64)
                host[r] = np.bincount(h[(h >= 0) & (h < vocab)], minlength=vocab)
            else:
                host[r] = 0
        self.counts.copy_(self.counts_host, non_blocking=True)
        bias: dict = {}
        for tok, b in options.logit_bias:
            bias[tok] = bias.get(tok, 0.0) + b
        dense = torch.zeros(vocab, dtype=torch.float32)
        for tok, b in bias.items():
            dense[tok] = b
        self.bias.copy_(dense)
        self.penalties.copy_(torch.tensor([options.repeat_penalty, options.presence_penalty, options.frequency_penalty],
                                          dtype=torch.float32))


class StepGraph:
    """A captured step of one layout with several tokens per sequence (prompts, chunks): the
    launches of such a step depend on the numbers of tokens, wanted places and block-table
    widths only, everything else reaches the kernels through the step's integer buffer. The step
    in which the layout comes back is run eagerly on this graph's own static buffers and then
    captured; later steps of the layout copy their integers and replay."""

    def __init__(self, model, cache, layout):
        dev = model.device
        self.model = model
        self.rows = layout.n_rows
        meta = torch.zeros(layout.total, dtype=torch.int32, device=dev)
        self.ctx = StepContext(cache=cache, workspace=Workspace(dev), dtype=model.dtype, device=dev, layout=layout,
                               meta_dev=meta, options=model.options)
        self.host = [torch.zeros(layout.total, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.events = [None] * _RING
        self.turn = 0
        self.graph = None
        self.logits = None
        self.launches = 0
        self.replays = 0

    def load(self, host_vec, slots, starts, news, row0) -> int:
        """The step's integers into the static buffer (one copy from pinned memory)."""
        i = self.turn
        self.turn = (self.turn + 1) % _RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        self.host[i].numpy()[:] = host_vec
        self.ctx.meta_dev.copy_(self.host[i], non_blocking=True)
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        self.ctx._set_host(slots, starts, news, row0)
        return host_vec.nbytes

    def run_and_capture(self) -> torch.Tensor:
        """This step for real, on the static buffers; then the capture (which runs nothing)."""
        out = self.model.run(self.ctx)
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.logits = self.model.run(self.ctx)
        self.launches = ops.launch_count() - before
        self.graph = g
        return out

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        self.replays += 1
        ops.add_launches(self.launches)
        return self.logits.clone()          # the next replay writes the same buffer
