"""The generation loop above the step function.

Requests are cut into batches that fit the cache; a batch starts together (all prompts in
one step, unequal lengths), then every live sequence goes on by one token per step. A
sequence ends on a stop token (which is kept, as the reference keeps its end-of-generation
token: src/main.rs:3731-3733, :3877-3879), on its token budget ("length",
src/api/mod.rs:11096, :11157) or when it has no room left in the cache or the model's
positions ("capacity", src/inference.rs:2660-2665). It leaves the batch at once and its slot
is given back; the next batch uses the slots again. Nothing joins a running batch.

The loop only decides; the model, the cache and the sampler are passed in, so its
decisions can be tested with stand-ins that need no device.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..cache.book import PAGE
from ..errors import CacheError, StepError
from .model import StepEntry


@dataclass
class GenerationResult:
    tokens: list = field(default_factory=list)       # generated ids, the stop token included
    finish_reason: str = ""                          # "stop", "length" or "capacity"
    prompt_tokens: int = 0


# Steps a greedy batch runs on the device between looks at its tokens when stop tokens are set.
FED_RUN_WITH_STOPS = 16


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


def token_budget(prompt_len: int, max_tokens: int, max_position: int, n_pages: int) -> int:
    """New tokens a request may produce: what was asked, cut to the model's positions and to
    a cache that it would have for itself."""
    room = min(max_position, n_pages * PAGE) - prompt_len + 1     # the last token is never fed back
    return max(0, min(max_tokens, room))


def plan_batches(prompt_lens: list, budgets: list, n_pages: int, n_slots: int, max_batch: int | None) -> list:
    """Cut the requests, in order, into batches whose sequences all fit the cache at their
    full length at the same time. Returns lists of request indices."""
    batches, cur, cur_pages = [], [], 0
    for i, (n, b) in enumerate(zip(prompt_lens, budgets)):
        need = pages_for(n + max(b - 1, 0))
        if need > n_pages:
            raise CacheError(f"request {i}: {n} prompt tokens need {need} pages, the cache has {n_pages}")
        limit = min(n_slots, max_batch or n_slots)
        if cur and (len(cur) >= limit or cur_pages + need > n_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


def _to_list(tokens) -> list:
    return tokens.tolist() if hasattr(tokens, "tolist") else list(tokens)


def run_batch(model, cache, sampler, prompts: list, budgets: list, requested: list, stop_ids: set,
              on_step=None) -> list:
    """One batch from its prompts to its last token. ``budgets[i]`` is the number of tokens
    sequence i may produce, ``requested[i]`` what was asked for (it decides between
    "length" and "capacity")."""
    n = len(prompts)
    results = [GenerationResult(prompt_tokens=len(p)) for p in prompts]
    slots = [None] * n
    histories = [list(p) for p in prompts]
    live = []
    try:
        for i in range(n):
            if budgets[i] <= 0:
                results[i].finish_reason = "capacity" if requested[i] > 0 else "length"
                continue
            slots[i] = cache.alloc_slot()
            live.append(i)
        if not live:
            return results
        entries = [StepEntry(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in live]
        # After the prompts, a model that steps through captured graphs and a sampler without
        # per-history adjustments hand the one-token steps to the C++ loop: many steps per call.
        native = (getattr(model, "use_graphs", False) and hasattr(model, "decode_natively")
                  and (getattr(sampler, "native_ok", False) or getattr(sampler, "fed_ok", False)))
        # Better still, the captured step picks the token itself (greedy, or sampled with a draw made
        # on the device from the seed and the row's position) and feeds it to the next step on the
        # device, so a run of steps is queued at once and read back at its end. Sequences do not depend on one another, so a sequence that meets a stop token
        # inside such a run just drops what it produced after it; with stop tokens the runs are
        # short, so that little is produced in vain.
        # Penalties and biases ride along there: the histories' token counts go to the device when a run starts.
        fed = (native and hasattr(model, "decode_fed")
               and getattr(getattr(model, "options", None), "feed_on_device", False))
        adjusts = bool(getattr(getattr(sampler, "options", None), "adjusts", False))
        if adjusts and not fed:
            native = False                                 # the C++ loop without feeding knows no adjustments
        first = True
        while live:
            if native and not first:
                k = min(budgets[i] - len(results[i].tokens) for i in live)
                if fed:
                    steps = min(k, FED_RUN_WITH_STOPS) if stop_ids else k
                    if adjusts:
                        out = model.decode_fed(cache, [slots[i] for i in live], [results[i].tokens[-1] for i in live],
                                               steps, sampler.options, histories=[histories[i] for i in live])
                    else:
                        out = model.decode_fed(cache, [slots[i] for i in live], [results[i].tokens[-1] for i in live],
                                               steps, sampler.options)
                else:
                    out, steps = model.decode_natively(cache, [slots[i] for i in live],
                                                       [results[i].tokens[-1] for i in live],
                                                       [len(histories[i]) for i in live], k, sorted(stop_ids),
                                                       sampler.options, sampler.error_word)
                still = []
                for j, i in enumerate(live):
                    new = [int(t) for t in out[:steps, j]]
                    for at, tok in enumerate(new):          # a run on the device goes on past a stop token
                        if tok in stop_ids:
                            new = new[:at + 1]
                            break
                    results[i].tokens.extend(new)
                    histories[i].extend(new)
                    if new[-1] in stop_ids:
                        results[i].finish_reason = "stop"
                    elif len(results[i].tokens) >= budgets[i]:
                        results[i].finish_reason = "length" if budgets[i] >= requested[i] else "capacity"
                    if results[i].finish_reason:
                        cache.free_slot(slots[i])
                        slots[i] = None
                    else:
                        still.append(i)
                if on_step is not None:
                    for _ in range(steps):
                        on_step(len(live))
                live = still
                continue
            first = False
            logits = model.step(cache, entries)
            tokens = _to_list(sampler.sample(logits, [histories[i] for i in live]))
            if on_step is not None:
                on_step(len(live))
            still, entries = [], []
            for i, tok in zip(live, tokens):
                tok = int(tok)
                results[i].tokens.append(tok)
                histories[i].append(tok)
                if tok in stop_ids:
                    results[i].finish_reason = "stop"
                elif len(results[i].tokens) >= budgets[i]:
                    results[i].finish_reason = "length" if budgets[i] >= requested[i] else "capacity"
                if results[i].finish_reason:
                    cache.free_slot(slots[i])
                    slots[i] = None
                else:
                    still.append(i)
                    entries.append(StepEntry(slots[i], [tok], [0]))
            live = still
    finally:
        for s in slots:
            if s is not None:
                cache.free_slot(s)
    return results


def generate(model, cache, sampler, prompts: list, max_tokens, *, stop_ids=(), max_batch: int | None = None,
             on_step=None) -> list:
    """Generate for every prompt; ``max_tokens`` is one number or one per prompt. Returns a
    ``GenerationResult`` per prompt, in the order given."""
    if not prompts:
        return []
    per = list(max_tokens) if isinstance(max_tokens, (list, tuple)) else [int(max_tokens)] * len(prompts)
    if len(per) != len(prompts):
        raise StepError("max_tokens must be one number or one per prompt")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise StepError(f"prompt {i} is empty")
        if per[i] < 0:
            raise StepError(f"prompt {i}: max_tokens must not be negative")
    book = cache.book
    lens = [len(p) for p in prompts]
    for i, n in enumerate(lens):
        if n > book.max_position:
            raise StepError(f"prompt {i}: {n} tokens exceed the model's {book.max_position} positions")
    budgets = [token_budget(n, m, book.max_position, book.n_pages) for n, m in zip(lens, per)]
    results = [None] * len(prompts)
    for batch in plan_batches(lens, budgets, book.n_pages, book.n_slots, max_batch):
        out = run_batch(model, cache, sampler, [list(prompts[i]) for i in batch], [budgets[i] for i in batch],
                        [per[i] for i in batch], set(stop_ids), on_step)
        for i, r in zip(batch, out):
            results[i] = r
    return results
