"""A model as data: which parts each layer is made of, and the order in which layers run.

An architecture turns its typed configuration into a ``ModelPlan``; the engine builds
the parts the plan names from the part registry (``camelid_b200.parts``) and knows
nothing else about the architecture. The reference's precedent is a per-layer plan
with a layer-kind switch inside one forward loop (src/model.rs:439-518).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered ``kind``, its sizes and constants, and the prefix of its
    tensors' names in the model folder (e.g. ``model.layers.3.self_attn.``)."""
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement of its parts (``prenorm``: x + mixer(norm(x)), then
    r + ffn(norm(r))) and the parts themselves. Layers of one model may differ."""
    arrangement: str
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``layer`` indexes ``ModelPlan.layers`` and may occur in several
    entries (the layer's weights are then shared, each entry keeping a cache of its own).
    ``cache_source`` names an earlier entry of the schedule whose keys and values this
    entry reads instead of making its own."""
    layer: int
    cache_source: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    embedding: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    hidden_size: int
    vocab_size: int
    max_position: int
    stop_token_ids: tuple = ()

    def __post_init__(self):
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError("schedule", f"schedule entry {i} names layer {e.layer}, the plan has {len(self.layers)}")
            if e.cache_source is not None:
                if not 0 <= e.cache_source < i:
                    raise ConfigError("schedule", f"schedule entry {i} reads the cache of entry {e.cache_source}, which does not run before it")
                if self.schedule[e.cache_source].cache_source is not None:
                    raise ConfigError("schedule", f"schedule entry {i} reads entry {e.cache_source}, which has no cache of its own")
