"""What a part is, and the registry the engine builds parts from.

A part is made from a ``PartSpec`` (its sizes and constants, and the prefix of its tensor
names). It says which tensors it needs (``tensor_specs``), takes them (``load``), and
runs on the rows of a step (``forward``; the signature depends on the role). No part knows
which model it is in: what it needs to know about the step comes with the ``StepContext``.

Roles and their ``forward``:

* ``norm``:      ``forward(ctx, h, rows_index=None, n_rows=None) -> x``; ``h`` is the float32
                 residual stream ``[rows, hidden]``, ``x`` has the compute type.
* ``mixer``:     ``forward(ctx, x, residual)``; adds its output into ``residual`` (float32) in
                 place. ``cache_spec()`` returns a ``KVSpec``, a ``StateSpec`` or None; the
                 storage of the running schedule entry is reached through ``ctx``.
* ``ffn``:       ``forward(ctx, x, residual)``; adds into ``residual`` in place.
* ``position``:  owned by a mixer; a rotary encoding exposes ``inv_freq`` and ``rotary_dim``.
* ``embedding``: ``forward(ctx, tokens, out)``; writes float32 rows.
* ``head``:      ``forward(ctx, x, out)``; writes float32 logits.
* ``block``:     the arrangement of norm, mixer, norm, feed-forward: ``forward(ctx, h)``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.plan import PartSpec
from ..errors import ConfigError

ROLES = ("norm", "mixer", "ffn", "position", "embedding", "head", "block")


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs: its shape and how random weights are drawn for it
    ("linear" and "embedding": N(0, 0.02); "norm": 1 + N(0, 0.02))."""
    shape: tuple
    init: str = "linear"


class Part:
    role: str = ""
    kind: str = ""
    # True if ``forward`` only launches work on the device arrays of the context (no host-side
    # reads of the step, no allocation that must outlive the call): such a part can run
    # inside a captured CUDA graph. Parts that do not say so make the model step eagerly.
    graph_safe: bool = False
    # True if that also holds for steps that bring several tokens per sequence (prompts): a model
    # whose parts all say so replays a captured graph for a step whose layout it has seen before.
    graph_safe_any_step: bool = False
    # True if the part knows what built-in parts may leave on the context instead of adding it
    # into the residual stream at once (``ctx.pending``: split sums; ``ctx.deferred``: a product
    # not yet launched) and deals with both itself. The block settles the stream before every
    # part that does not say so: a part from outside the library always sees complete rows.
    handles_pending: bool = False
    # True if ``forward`` takes ``ctx.take_row_scale()`` before it reads its input rows and
    # applies the scale itself (to the rows, or to the output of a product of them). The norm
    # before such a part may then leave its rows' scale to the part.
    accepts_row_scale: bool = False

    def __init__(self, params: dict, prefix: str = ""):
        self.params = dict(params)
        self.prefix = prefix

    def tensor_specs(self) -> dict:
        """Full tensor name -> TensorSpec."""
        return {}

    def load(self, tensors: dict, device, dtype: torch.dtype) -> None:
        """Take the tensors named by ``tensor_specs`` (CPU or device) to the device."""

    def cache_spec(self):
        return None

    def query_tile_sizes(self) -> list:
        """Mixers: the sizes of query tiles (rows per tile) their prefill kernels ask the
        step context for."""
        return []


_REGISTRY: dict = {role: {} for role in ROLES}


def register_part(role: str, kind: str):
    """Class decorator: ``@register_part("mixer", "attention")``. A later registration of the
    same name replaces the earlier one."""
    if role not in _REGISTRY:
        raise ConfigError("role", f"unknown role {role!r}; roles are {ROLES}")

    def deco(cls):
        cls.role, cls.kind = role, kind
        _REGISTRY[role][kind] = cls
        return cls
    return deco


def known_parts(role: str) -> list:
    return sorted(_REGISTRY[role])


def build_part(role: str, spec: PartSpec):
    try:
        cls = _REGISTRY[role][spec.kind]
    except KeyError:
        raise ConfigError(f"{role}.kind", f"no {role} named {spec.kind!r} is registered; known: {known_parts(role)}") from None
    return cls(spec.params, spec.prefix)


def build_block(layer_spec):
    """The arrangement a ``LayerSpec`` names, built with the layer's parts."""
    try:
        cls = _REGISTRY["block"][layer_spec.arrangement]
    except KeyError:
        raise ConfigError("block.arrangement", f"no block arrangement named {layer_spec.arrangement!r} is registered; "
                          f"known: {known_parts('block')}") from None
    return cls(layer_spec)


def to_device(t: torch.Tensor, device, dtype: torch.dtype | None) -> torch.Tensor:
    """Copy a weight to the device. ``dtype`` None keeps the stored type."""
    if dtype is not None and t.dtype != dtype:
        if t.is_cuda or t.numel() < (1 << 22):
            return t.to(device=device, dtype=dtype).contiguous()
        return t.to(device=device).to(dtype).contiguous()        # convert on the device, not on the host
    return t.to(device=device).contiguous()
