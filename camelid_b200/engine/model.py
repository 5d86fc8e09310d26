"""The model as the engine sees it: parts built from a plan, and one step function.

``step`` takes a batch of sequences with unequal numbers of new tokens (whole prompts in
one step, then one token each; any mix works, since every row carries its own position),
runs exactly those tokens as one packed batch against the cache, and returns the float32
logits at the wanted places. Every check happens before any device work, so a refused
step leaves the cache as it was (the reference's precedent: tests/inference_session.rs:409-543).

The reference's counterparts are the session's ``generate_next_token`` path
(src/inference.rs:4383-4548) with ``forward_prefill_chunk_timed_fast`` (:3657-3751) and
the resident engine's ``forward_pass_inner`` / ``run_batched_layer_stack``
(src/cuda_resident.rs:6445-7426, :7975-8289); logits only where asked follows
``forward_final_norm_and_logits`` (src/inference.rs:3638-3651).
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.sequence_cache import SequenceCache
from ..config.plan import ModelPlan
from ..config.registry import load_config
from ..errors import ConfigError, KernelError, StepError
from ..options import KernelOptions
from ..parts import build_block, build_part
from ..weights.loader import check_tensors
from ..weights.safetensors_io import ModelFiles
from .context import StepContext, Workspace

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ConfigError("dtype", f"the compute type must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ConfigError("dtype", f"the compute type must be 'bfloat16' or 'float32', got {dtype!r}") from None


@dataclass
class StepEntry:
    """One sequence of a step: its slot, its next tokens, and the places among these tokens
    (0-based) whose logits are wanted."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)


class DecoderModel:
    def __init__(self, plan: ModelPlan, *, dtype=torch.bfloat16, device="cuda", typed_config=None,
                 options: KernelOptions | None = None):
        self.plan = plan
        self.typed_config = typed_config
        self.options = options if options is not None else KernelOptions()
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        self.embedding = build_part("embedding", plan.embedding)
        self.blocks = [build_block(layer) for layer in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.schedule = list(plan.schedule)
        self.hidden_size = plan.hidden_size
        self.vocab_size = plan.vocab_size
        self.loaded = False
        self.workspace = Workspace(self.device)
        self._err = None
        self._logit_err = None
        self.last_h2d_bytes = 0
        self.tile_sizes = sorted({r for b in self.blocks for r in b.query_tile_sizes()}) or [1]
        # decode steps replay captured CUDA graphs when every part can run inside one
        self.use_graphs = all(b.graph_safe for b in self.blocks) and all(
            p.graph_safe for p in (self.embedding, self.final_norm, self.head))
        self._graphs = weakref.WeakKeyDictionary()      # cache -> {(sequences, widths, feed): DecodeGraph}
        # steps of several tokens per sequence: layouts seen once, and the graphs of those seen again
        self.capture_steps = (self.use_graphs and self.options.capture_repeated_steps
                              and all(b.graph_safe_any_step for b in self.blocks)
                              and all(p.graph_safe_any_step for p in (self.embedding, self.final_norm, self.head)))
        self._seen_layouts = weakref.WeakKeyDictionary()   # cache -> {key: times seen}
        self._step_graphs = weakref.WeakKeyDictionary()    # cache -> {key: StepGraph}, oldest first

    # ---- construction ----
    @classmethod
    def from_config(cls, config, *, dtype=torch.bfloat16, device="cuda", options=None) -> "DecoderModel":
        """``config``: a config.json dict or a model folder. Builds the parts; no weights yet."""
        _arch, typed, plan = load_config(config)
        return cls(plan, dtype=dtype, device=device, typed_config=typed, options=options)

    @classmethod
    def from_folder(cls, folder: str, *, dtype=torch.bfloat16, device="cuda", options=None) -> "DecoderModel":
        model = cls.from_config(folder, dtype=dtype, device=device, options=options)
        files = ModelFiles(folder)
        try:
            model.load_tensors(files)
        finally:
            files.close()
        return model

    def tensor_specs(self) -> dict:
        specs = dict(self.embedding.tensor_specs())
        for b in self.blocks:
            specs.update(b.tensor_specs())
        specs.update(self.final_norm.tensor_specs())
        specs.update(self.head.tensor_specs())
        return specs

    def memory_plan(self, max_tokens: int = 0, max_slots: int | None = None, step_tokens: int | None = None):
        from ..memory import plan_for_model
        return plan_for_model(self, max_tokens, max_slots, step_tokens)

    def load_tensors(self, source, available_bytes: int | None = None) -> None:
        """``source``: ``ModelFiles`` or a dict name -> tensor. Checks names and shapes first, then
        that the weights fit the device's free memory (``available_bytes`` stands in for it)."""
        specs = self.tensor_specs()
        if isinstance(source, dict):
            found = {n: (tuple(t.shape), t.dtype) for n, t in source.items()}
            get = source.__getitem__
        else:
            found = {n: (tuple(source.shape(n)), source.dtype(n)) for n in source.names()}
            get = source.tensor
        tied = getattr(self.head, "tied_to", None)
        tolerated = (self.head.prefix + "weight",) if tied else ()
        check_tensors(specs, found, tolerated=tolerated)
        from ..memory import device_free_bytes
        free = available_bytes if available_bytes is not None else device_free_bytes(self.device)
        if free is not None:
            held = sum(t.numel() * t.element_size() for t in source.values() if t.is_cuda) if isinstance(source, dict) else 0
            self.memory_plan().check(free + held, f"loading the weights onto {self.device}", parts=("weights",))

        class _Lazy(dict):
            def __missing__(self, name):
                return get(name)
        tensors = _Lazy()
        self.embedding.load(tensors, self.device, self.dtype)
        for b in self.blocks:
            b.load(tensors, self.device, self.dtype)
        self.final_norm.load(tensors, self.device, self.dtype)
        if tied:
            self.head.load(tensors, self.device, self.dtype, tied_weight=self.embedding.weight)
        else:
            self.head.load(tensors, self.device, self.dtype)
        self.loaded = True

    # ---- cache ----
    def entry_cache_specs(self) -> list:
        return [self.blocks[e.layer].cache_spec() for e in self.schedule]

    def new_cache(self, max_tokens: int, max_slots: int | None = None) -> SequenceCache:
        """A cache for at most ``max_tokens`` live tokens (each sequence's count rounded up to
        a multiple of 64) and ``max_slots`` live sequences (default: one per page)."""
        from ..memory import device_free_bytes
        free = device_free_bytes(self.device)
        if free is not None:
            self.memory_plan(max_tokens, max_slots).check(free, f"a cache for {max_tokens} tokens on {self.device}",
                                                          parts=("cache", "workspace"))
        return SequenceCache(self.entry_cache_specs(), [e.cache_source for e in self.schedule],
                             max_tokens=max_tokens, max_position=self.plan.max_position, dtype=self.dtype,
                             device=self.device, max_slots=max_slots)

    # ---- the step ----
    def _validate(self, cache: SequenceCache, entries: list) -> list:
        """Checks a step before anything changes; returns each entry's tokens as an int64 array."""
        if not self.loaded:
            raise StepError("the model has no weights yet")
        if self.device.type != "cuda":
            raise KernelError("steps run on a CUDA device only; there is no CPU path")
        if not entries:
            raise StepError("a step needs at least one sequence")
        arrays = []
        for e in entries:
            try:
                a = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
            except (TypeError, ValueError, OverflowError):
                raise StepError(f"slot {e.slot}: the tokens are not a flat sequence of integer ids") from None
            if a.size == 0:
                raise StepError(f"slot {e.slot}: a step must bring at least one token")
            if int(a.min()) < 0 or int(a.max()) >= self.vocab_size:
                bad = int(a[(a < 0) | (a >= self.vocab_size)][0])
                raise StepError(f"slot {e.slot}: token id {bad} is outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < a.size:
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside the step's {a.size} tokens")
            arrays.append(a)
        cache.book.check_extend([(e.slot, a.size) for e, a in zip(entries, arrays)])
        return arrays

    def step(self, cache: SequenceCache, entries: list) -> torch.Tensor:
        """Run the given tokens; returns float32 logits [wanted places, vocabulary] in the order
        of the entries and of their ``want`` lists (an empty tensor if nothing is wanted)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        arrays = self._validate(cache, entries)
        if self.use_graphs and all(a.size == 1 and list(e.want) == [0] for e, a in zip(entries, arrays)):
            return self._graph_step(cache, entries)
        starts = [cache.book.extend(e.slot, a.size) for e, a in zip(entries, arrays)]
        slots = [e.slot for e in entries]
        want = [[int(w) for w in e.want] for e in entries]
        logits = None
        if self.capture_steps and max(a.size for a in arrays) > 1:
            logits = self._captured_step(cache, slots, starts, arrays, want)
        if logits is None:
            ctx = StepContext.for_step(cache=cache, workspace=self.workspace, dtype=self.dtype, device=self.device,
                                       slots=slots, starts=starts, tokens=arrays, want=want, tile_sizes=self.tile_sizes,
                                       options=self.options)
            logits = self.run(ctx)
            self.last_h2d_bytes = ctx.h2d_bytes
        for e, a in zip(entries, arrays):
            cache.book.commit(e.slot, a.size)
        return logits

    def _captured_step(self, cache, slots, starts, arrays, want):
        """The step through a captured graph if its layout was seen before (None: run it eagerly).
        The layout is what the launches depend on: tokens per sequence, the number of wanted
        places and the block-table widths."""
        from .graphs import StepGraph
        book = cache.book
        tables = [book.block_table(g, slots) for g in range(len(book.kv_specs))]
        key = (tuple(int(a.size) for a in arrays), sum(len(w) for w in want), tuple(len(t[0]) for t in tables))
        graphs = self._step_graphs.setdefault(cache, {})
        graph = graphs.get(key)
        seen = self._seen_layouts.setdefault(cache, {})         # how often each layout has come by
        if len(seen) > 4096:
            seen.clear()
        seen[key] = seen.get(key, 0) + 1
        if graph is None:
            # A capture costs tens to hundreds of milliseconds and saves a fraction of one per replay, less the
            # longer the step: a layout is captured when it comes back (the third time for a long step), and only
            # if there is room for it after dropping graphs of layouts that have come by less often than this
            # one (the least recently used first). Layouts that take turns, more of them than the kept rows
            # hold, have come by equally often: the first ones keep their graphs, the others run eagerly,
            # instead of each being captured and dropped in turn for ever.
            rows = sum(int(a.size) for a in arrays)
            if seen[key] < (2 if rows <= 512 else 3) or rows > self.options.captured_step_rows:
                return None
            room = self.options.captured_step_rows - sum(g.rows for g in graphs.values())
            drop = []
            for k, g in graphs.items():                          # least recently used first
                if room >= rows:
                    break
                if seen.get(k, 0) < seen[key]:
                    drop.append(k)
                    room += g.rows
            if room < rows:
                return None
            for k in drop:
                del graphs[k]
        layout, host, news, row0 = StepContext.host_arrays(slots, starts, arrays, want, tables, self.tile_sizes)
        if graph is None:
            graph = StepGraph(self, cache, layout)
            self.last_h2d_bytes = graph.load(host, slots, starts, news, row0)
            logits = graph.run_and_capture()
            graphs[key] = graph
            return logits
        graphs[key] = graphs.pop(key)                           # most recently used last
        self.last_h2d_bytes = graph.load(host, slots, starts, news, row0)
        return graph.replay()

    MAX_DECODE_GRAPHS = 128     # per cache: batch sizes times block-table widths times the ways a step picks its token

    def decode_graph(self, cache: SequenceCache, slots: list, feed: bool = False, adjust: bool = False):
        """The captured graph for one-token steps of these slots (made at its first use)."""
        from .graphs import DecodeGraph, bucket_width
        book = cache.book
        widths = [bucket_width(max(len(book.pages[g][s]) for s in slots)) for g in range(len(book.kv_specs))]
        graphs = self._graphs.setdefault(cache, {})
        key = (len(slots), tuple(widths), feed, adjust)
        graph = graphs.pop(key, None)
        if graph is None:
            graph = DecodeGraph(self, cache, len(slots), widths, feed, adjust)
            while len(graphs) >= self.MAX_DECODE_GRAPHS:        # each holds its own buffers: the least recently used goes
                del graphs[next(iter(graphs))]
        graphs[key] = graph                                     # most recently used last
        return graph

    def decode_natively(self, cache: SequenceCache, slots: list, tokens: list, history_lens: list, max_steps: int,
                        stop_ids, options, err: torch.Tensor) -> tuple:
        """Run up to ``max_steps`` one-token steps of these sequences in the C++ loop: each feeds
        its token, the sampling kernel picks the next, which is fed in the next step. Stops after
        the step in which a sequence picks a stop token. Returns (tokens [steps][sequence], steps);
        the cache's lengths have moved by ``steps``."""
        if self._err is None:
            self._err = torch.zeros(1, dtype=torch.int32, device=self.device)
        if not self.use_graphs:
            raise StepError("the C++ decode loop needs a model whose parts can run in a captured graph")
        for t in tokens:
            if not 0 <= int(t) < self.vocab_size:
                raise StepError(f"token id {t} is outside the vocabulary of {self.vocab_size}")
        book = cache.book
        book.check_extend([(s, max_steps) for s in slots])
        starts = [book.extend(s, max_steps) for s in slots]
        graph = self.decode_graph(cache, slots)
        out, steps = graph.run_native(slots, starts, [int(t) for t in tokens], history_lens, max_steps, stop_ids,
                                      options.temperature, options.top_k, options.top_p, options.min_p, options.seed, err)
        for s in slots:
            book.commit(s, steps)
        self.last_h2d_bytes = graph.native_loop(err).h2d_bytes_per_step
        return out, steps

    def logit_error_word(self) -> torch.Tensor:
        """int32[1] on the device: set by the greedy choice inside a captured step when a logit is
        not finite; ``check_device_errors`` reads it."""
        if self._logit_err is None:
            self._logit_err = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._logit_err

    def decode_fed(self, cache: SequenceCache, slots: list, tokens: list, steps: int, sampling=None, histories=None):
        """Exactly ``steps`` one-token steps of these sequences with the chosen token fed back on the
        device: all steps are queued at once and the host waits once at the end. ``sampling``
        (``SamplingOptions``; None or temperature 0: greedy): the draws are made on the device from the
        seed and each row's position, the same numbers the host would draw. With penalties or a bias,
        ``histories`` gives per sequence the tokens so far (the one fed first included): their counts
        go to the device once and the steps count what they choose. Returns the tokens
        [steps][sequence] (numpy); the cache's lengths have moved by ``steps``."""
        if not self.use_graphs:
            raise StepError("decoding with the token fed back on the device needs a model whose parts can run in a captured graph")
        if not self.loaded:
            raise StepError("the model has no weights yet")
        for t in tokens:
            if not 0 <= int(t) < self.vocab_size:
                raise StepError(f"token id {t} is outside the vocabulary of {self.vocab_size}")
        if steps <= 0:
            raise StepError("decode_fed needs at least one step")
        adjust = sampling is not None and sampling.adjusts
        if adjust and (histories is None or len(histories) != len(slots)):
            raise StepError("penalties and biases need each sequence's history: pass histories to decode_fed")
        book = cache.book
        book.check_extend([(s, steps) for s in slots])
        starts = [book.extend(s, steps) for s in slots]
        feed, seed = True, 0
        if sampling is not None and not sampling.greedy:
            feed = "sample"              # temperature and filters reach the kernel through device memory
            seed = int(sampling.seed or 0)
        graph = self.decode_graph(cache, slots, feed=feed, adjust=adjust)
        out = graph.run_fed(slots, starts, [int(t) for t in tokens], steps, seed, histories, sampling)
        for s in slots:
            book.commit(s, steps)
        self.last_h2d_bytes = graph._fed.h2d_bytes_per_step
        return out

    def drop_graphs(self, cache=None) -> None:
        """Forget the captured graphs of one cache, or all. (A cache that is no longer referenced
        takes its graphs with it: they are kept per cache and hold no reference to it.)"""
        for kept in (self._graphs, self._step_graphs, self._seen_layouts):
            if cache is None:
                kept.clear()
            else:
                kept.pop(cache, None)

    def _graph_step(self, cache: SequenceCache, entries: list) -> torch.Tensor:
        slots = [e.slot for e in entries]
        starts = [cache.book.extend(s, 1) for s in slots]
        graph = self.decode_graph(cache, slots)
        i = graph.fill(slots, starts, [int(e.tokens[0]) for e in entries])
        self.last_h2d_bytes = graph.send(i, with_tokens=True)
        if graph.graph is None:
            graph.capture()
        logits = graph.replay()
        for s in slots:
            cache.book.commit(s, 1)
        return logits

    def run(self, ctx: StepContext) -> torch.Tensor:
        """The forward pass of one step on a prepared context."""
        from ..csrc import ops
        ops.set_dependent_launch(self.options.dependent_launch)
        if self._err is None:
            self._err = torch.zeros(1, dtype=torch.int32, device=self.device)
        ctx.pending = None
        ctx.deferred = None
        ctx.row_scale = None
        h = ctx.buffer("hidden", (ctx.n_rows, self.hidden_size), torch.float32)
        self.embedding.forward(ctx, ctx.tokens, h, self._err)
        for i, e in enumerate(self.schedule):
            ctx.entry = i
            ctx.cache_source = e.cache_source
            self.blocks[e.layer].forward(ctx, h)
        logits = torch.empty((ctx.n_want, self.vocab_size), dtype=torch.float32, device=self.device)
        if ctx.n_want:
            if not self.final_norm.handles_pending:          # a norm from outside reads a settled stream
                ctx.settle(h)
            x = self.final_norm.forward(ctx, h, rows_index=ctx.want_rows, n_rows=ctx.n_want, name="final_normed")
            self.head.forward(ctx, x, logits)
        ctx.pending = None
        ctx.deferred = None
        return logits

    def check_device_errors(self) -> None:
        """Reads the device-side error word (a synchronising copy) and raises if a kernel saw
        a token id outside the vocabulary."""
        if self._err is not None and int(self._err.item()) != 0:
            self._err.zero_()
            raise StepError("a kernel met a token id outside the vocabulary")
        if self._logit_err is not None and int(self._logit_err.item()) != 0:
            self._logit_err.zero_()
            from ..errors import SamplingError
            raise SamplingError("the logits of a step that chose its tokens on the device contain a non-finite value "
                                "(or its softmax sum was not a positive number)")
        from ..parts import linear
        linear.check_errors()
