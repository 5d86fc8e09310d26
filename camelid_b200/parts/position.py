"""Position encodings. The rotary one owns its per-pair frequencies; the mixer's kernel
turns position * frequency into sine and cosine in float32 and rotates split-half pairs.

Frequencies as the reference computes them, in float32: f_i = theta^(-2i / rotary_dim)
(src/inference/rope.rs:526-537), then for ``llama3`` scaling: wavelength = 2 pi / f; below
original/high the frequency stays, above original/low it is divided by the factor, between
them it is blended with smooth = (original / wavelength - low) / (high - low)
(src/inference/rope.rs:687-711)."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..errors import ConfigError
from .base import Part, register_part


def rotary_frequencies(rotary_dim: int, theta: float, scaling: dict | None) -> np.ndarray:
    f32 = np.float32
    idx = np.arange(rotary_dim // 2, dtype=np.float32)
    expo = (-(idx * f32(2.0)) / f32(rotary_dim)).astype(np.float32)
    freq = np.power(f32(theta), expo).astype(np.float32)
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            factor = f32(scaling["factor"])
            low = f32(scaling.get("low_freq_factor", 1.0))
            high = f32(scaling.get("high_freq_factor", 4.0))
            orig = f32(scaling.get("original_max_position_embeddings", 8192))
            wavelength = (f32(2.0) * f32(math.pi)) / freq
            smooth = ((orig / wavelength - low) / (high - low)).astype(np.float32)
            blended = ((f32(1.0) - smooth) * freq / factor + smooth * freq).astype(np.float32)
            freq = np.where(wavelength < orig / high, freq,
                            np.where(wavelength > orig / low, (freq / factor).astype(np.float32), blended)).astype(np.float32)
        elif kind not in (None, "default"):
            raise ConfigError("scaling.rope_type", f"rotary scaling {kind!r} is not known to this position encoding")
    return freq


@register_part("position", "rope")
class RotaryEncoding(Part):
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim % 2:
            raise ConfigError("rotary_dim", f"must be even, got {self.rotary_dim}")
        self.theta = float(params["theta"])
        self.scaling = params.get("scaling")
        self.inv_freq = None

    def load(self, tensors, device, dtype):
        self.inv_freq = torch.from_numpy(rotary_frequencies(self.rotary_dim, self.theta, self.scaling)).to(device)


@register_part("position", "none")
class NoPositionEncoding(Part):
    """Leaves q and k as they are: a rotary encoding of zero dimensions."""
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.rotary_dim = 0
        self.inv_freq = None

    def load(self, tensors, device, dtype):
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)
