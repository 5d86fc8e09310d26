"""What a model will hold on the device, worked out before anything is allocated.

``memory_plan`` needs no device: from a configuration, a compute type and the size of the
cache it gives the bytes of the weights, of the cache, and of the workspace a step of a given
size uses, so that a caller can ask first and the library can refuse with the numbers instead
of running into the allocator in the middle of a load. ``load`` / ``from_random`` check the
weights against the device's free memory, ``new_cache`` the cache and a step's workspace.

The reference sizes its cache from the model's dimensions (``ModelDims``, ``kv_bytes``:
src/fit.rs:253-298) and refuses a growth that would pass its budget before allocating
(src/inference/kv_cache.rs:285-299, VRAM sizing at src/inference.rs:11310-11330); its
allowance for activations is a fixed 512 MiB, here it follows the step's rows.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .cache.book import PAGE, KVSpec, StateSpec
from .errors import CacheError


class MemoryBudgetError(CacheError):
    """The plan does not fit the memory that is available; carries both."""

    def __init__(self, what: str, plan: "MemoryPlan", needed: int, available: int):
        self.plan, self.needed, self.available = plan, int(needed), int(available)
        super().__init__(f"{what}: {needed:,} bytes are needed, {available:,} are available "
                         f"(weights {plan.weights:,}, cache {plan.cache:,}, workspace {plan.workspace:,})")


@dataclass(frozen=True)
class MemoryPlan:
    weights: int          # every tensor the model keeps, in the compute type (norm weights as stored)
    cache: int            # keys, values and fixed-size state for max_tokens / max_slots
    workspace: int        # activations, split sums and logits of one step of step_tokens rows
    max_tokens: int
    max_slots: int
    step_tokens: int

    @property
    def total(self) -> int:
        return self.weights + self.cache + self.workspace

    def as_dict(self) -> dict:
        return {"weights": self.weights, "cache": self.cache, "workspace": self.workspace, "total": self.total}

    def check(self, available: int, what: str = "the model", parts=("weights", "cache", "workspace")) -> None:
        """Raise ``MemoryBudgetError`` if the named parts together pass ``available`` bytes."""
        needed = sum(getattr(self, p) for p in parts)
        if needed > available:
            raise MemoryBudgetError(what, self, needed, available)


def _elem(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def plan_for_model(model, max_tokens: int = 0, max_slots: int | None = None, step_tokens: int | None = None) -> MemoryPlan:
    """The plan of a built (not necessarily loaded) ``DecoderModel``; no device is touched."""
    e = _elem(model.dtype)
    specs = model.tensor_specs()
    weights = sum(_numel(s.shape) * e for s in specs.values())
    n_pages = max(1, (int(max_tokens) + PAGE - 1) // PAGE) if max_tokens else 0
    n_slots = int(max_slots) if max_slots else n_pages
    cache = 0
    seen_sources = [src for src in (entry.cache_source for entry in model.schedule)]
    widest_kv = 0
    for spec, src in zip(model.entry_cache_specs(), seen_sources):
        if src is not None or spec is None:
            continue
        if isinstance(spec, KVSpec):
            cache += 2 * n_pages * spec.n_kv_heads * PAGE * spec.head_dim * e
            widest_kv = max(widest_kv, spec.n_kv_heads * spec.head_dim)
        elif isinstance(spec, StateSpec):
            from .cache.sequence_cache import _STATE_DTYPES
            cache += n_slots * _numel(spec.shape) * _elem(_STATE_DTYPES[spec.dtype])
    rows = int(step_tokens) if step_tokens else min(max(int(max_tokens), 1), 2048)
    hidden = model.hidden_size
    widest = max([hidden] + [_numel(s.shape) // max(1, s.shape[-1]) for s in specs.values() if len(s.shape) == 2
                             and s.shape[0] != model.vocab_size])
    # one step: the float32 residual stream, the normed rows, q/k/v, the attention output and the
    # widest activation in the compute type; float32 split sums of one product (up to 8 splits of
    # the rows that decode paths take, 4 of a wide step); float32 logits of one row per sequence
    per_row = 4 * hidden + e * (2 * hidden + 2 * widest + 2 * widest_kv)
    partial_rows = min(rows, 128)
    workspace = rows * per_row + 4 * 4 * rows * hidden + 8 * 4 * partial_rows * widest
    workspace += 4 * max(n_slots, 1) * model.vocab_size
    return MemoryPlan(int(weights), int(cache), int(workspace), int(max_tokens), int(n_slots), int(rows))


def memory_plan(config, dtype="bfloat16", max_tokens: int = 0, max_slots: int | None = None,
                step_tokens: int | None = None) -> MemoryPlan:
    """``config``: a config.json dict or a model folder. Bytes of weights, cache (for
    ``max_tokens`` live tokens, each sequence's count rounded up to 64, and ``max_slots``
    sequences) and workspace (a step of ``step_tokens`` rows; default the smaller of
    ``max_tokens`` and 2,048). Runs without a device."""
    from .engine.model import DecoderModel, parse_dtype
    model = DecoderModel.from_config(config, dtype=parse_dtype(dtype), device="cpu")
    return plan_for_model(model, max_tokens, max_slots, step_tokens)


def device_free_bytes(device) -> int | None:
    """Free bytes on a CUDA device (memory this process's allocator holds but does not use
    counts as free); None where there is no such device."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return None
    free, _total = torch.cuda.mem_get_info(device)
    reserved = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    return int(free + max(0, reserved))
