"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same tensors drawn straight on the device.

Linear and embedding matrices are N(0, 0.02), norm weights 1 + N(0, 0.02), from the
library's counter-based generator (``counter_random``): a tensor's values depend on the seed
and on its own name only, and element ``i`` is the same number on the host and on the
device, bit for bit. So a folder written on the CPU and a model drawn on the GPU with the
same configuration and seed hold the same weights, and any slice of a large model can be
recomputed on the host. bfloat16 storage rounds the float32 draw. The reference has random
weights only in tests (an LCG: src/cuda_resident/tests.rs:537-553, norms 1 + 0.2u at
:217-224).
"""
from __future__ import annotations

import json
import os

import torch

from . import counter_random
from .safetensors_io import write_safetensors

STD = 0.02


def mean_of(init: str) -> float:
    return 1.0 if init == "norm" else 0.0


def random_slice(name: str, init: str, seed: int, first: int, count: int) -> torch.Tensor:
    """float32 values of elements ``first .. first + count`` (row-major) of tensor ``name``,
    computed on the host."""
    key = counter_random.tensor_key(seed, name)
    return torch.from_numpy(counter_random.fill_host(key, first, count, mean_of(init), STD))


def random_tensor(name: str, spec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    shape = tuple(int(s) for s in spec.shape)
    if torch.device(device).type == "cuda":
        from ..csrc import ops
        out = torch.empty(shape, dtype=dtype, device=device)
        ops.random_fill(out, counter_random.tensor_key(seed, name), 0, mean_of(spec.init), STD)
        return out
    n = 1
    for s in shape:
        n *= s
    return random_slice(name, spec.init, seed, 0, n).reshape(shape).to(dtype)


def random_tensors(specs: dict, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                   norm_dtype: torch.dtype | None = None) -> dict:
    """name -> tensor for every wanted tensor. ``norm_dtype`` stores norm weights in another
    type than the matrices (checkpoints keep them in 32-bit at times)."""
    return {n: random_tensor(n, s, seed, norm_dtype if (norm_dtype is not None and s.init == "norm") else dtype, device)
            for n, s in specs.items()}


def write_random_model(folder: str, config: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       norm_dtype: torch.dtype | None = None, device="cpu") -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for the architecture that
    ``config`` (a config.json dict) names. ``device``: where the numbers are drawn (the same
    numbers either way; a GPU draws a billion of them in a moment, the host takes a minute)."""
    from ..engine.model import DecoderModel          # late: the engine imports this package
    model = DecoderModel.from_config(config, dtype=dtype, device="cpu")
    tensors = {n: t.cpu() for n, t in random_tensors(model.tensor_specs(), seed, dtype, device, norm_dtype).items()}
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(model.typed_config.to_dict() if hasattr(model.typed_config, "to_dict") else config, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed, "generator": "camelid_b200.weights.counter_random"})
    return folder
