"""Helpers of the tests: tolerances, the oracle's logits, token sequences."""
import numpy as np
import torch

import plain_llama as pl

# Largest absolute difference of logits, relative to the largest reference logit of the
# compared block. float32: rounding of sums of a few thousand products. bfloat16: 8 bits of
# mantissa at every stored activation, through all layers.
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


def rel_err(got, ref) -> float:
    got = torch.as_tensor(got, dtype=torch.float64)
    ref = torch.as_tensor(ref, dtype=torch.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), "engine logits are not finite"
    return float((got - ref).abs().max() / max(float(ref.abs().max()), 1e-12))


def assert_close(got, ref, dtype: str, what: str = ""):
    e = rel_err(got, ref)
    assert e <= TOL[dtype], f"{what}: relative error {e:.3e} exceeds {TOL[dtype]:.1e} ({dtype})"


_oracle_cache: dict = {}


def oracle(folder: str, ids, schedule=None) -> torch.Tensor:
    """float64 logits [T, V] of the plain implementation for one whole sequence."""
    key = (folder, tuple(int(i) for i in ids), None if schedule is None else tuple(schedule))
    if key not in _oracle_cache:
        cfg, w = pl.read_model(folder)
        _oracle_cache[key] = pl.forward(cfg, w, list(ids), dtype=torch.float64, schedule=schedule)
    return _oracle_cache[key]


def tokens(seed: int, n: int, vocab: int) -> list:
    rng = np.random.default_rng(seed)
    return [int(x) for x in rng.integers(0, vocab, size=n)]
