"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

Linear and embedding matrices are N(0, 0.02), norm weights 1 + N(0, 0.02); every tensor
has a generator of its own, seeded by the seed and the tensor's name, so a tensor's values
do not depend on which other tensors the model has. The reference has random weights only
in tests (an LCG: src/cuda_resident/tests.rs:537-553, norms 1 + 0.2u at :217-224).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .safetensors_io import write_safetensors

STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    t = torch.randn(tuple(spec.shape), generator=gen, dtype=torch.float32, device=device) * STD
    if spec.init == "norm":
        t = t + 1.0
    return t.to(dtype)


def random_tensors(specs: dict, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                   norm_dtype: torch.dtype | None = None) -> dict:
    """name -> tensor for every wanted tensor. ``norm_dtype`` stores norm weights in another
    type than the matrices (checkpoints keep them in 32-bit at times)."""
    return {n: random_tensor(n, s, seed, norm_dtype if (norm_dtype is not None and s.init == "norm") else dtype, device)
            for n, s in specs.items()}


def write_random_model(folder: str, config: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       norm_dtype: torch.dtype | None = None) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for the architecture that
    ``config`` (a config.json dict) names."""
    from ..engine.model import DecoderModel          # late: the engine imports this package
    model = DecoderModel.from_config(config, dtype=dtype, device="cpu")
    tensors = random_tensors(model.tensor_specs(), seed, dtype, "cpu", norm_dtype)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(model.typed_config.to_dict() if hasattr(model.typed_config, "to_dict") else config, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed, "generator": "camelid_b200.weights.random_init"})
    return folder
