"""Helpers of the tests: tolerances, the oracle's logits, token sequences."""
import numpy as np
import torch

import plain_llama as pl

# Largest absolute difference of logits, relative to the largest reference logit: over the
# compared block, and for every row against that row's own largest logit (so that an error
# in one row cannot hide behind a large logit of another). float32: rounding of sums of a few
# thousand products. bfloat16: 8 bits of mantissa at every stored activation, through all layers.
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
# Mean absolute difference over the block, relative to its largest reference logit: rounding
# errors are spread evenly and stay an order of magnitude below the worst one; an error that
# touches every logit a little (a scale, a dropped key among thousands) shows here first.
MEAN_TOL = {"float32": 1e-5, "bfloat16": 4e-3}


def rel_err(got, ref) -> float:
    got = torch.as_tensor(got, dtype=torch.float64)
    ref = torch.as_tensor(ref, dtype=torch.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), "engine logits are not finite"
    return float((got - ref).abs().max() / max(float(ref.abs().max()), 1e-12))


def row_errors(got, ref) -> torch.Tensor:
    """For every row: largest absolute difference over the row's own largest reference logit."""
    got = torch.as_tensor(got, dtype=torch.float64).reshape(-1, got.shape[-1])
    ref = torch.as_tensor(ref, dtype=torch.float64).reshape(-1, ref.shape[-1])
    return (got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-12)


def mean_err(got, ref) -> float:
    got = torch.as_tensor(got, dtype=torch.float64)
    ref = torch.as_tensor(ref, dtype=torch.float64)
    return float((got - ref).abs().mean() / max(float(ref.abs().max()), 1e-12))


def assert_close(got, ref, dtype: str, what: str = ""):
    e = rel_err(got, ref)
    assert e <= TOL[dtype], f"{what}: relative error {e:.3e} exceeds {TOL[dtype]:.1e} ({dtype})"
    if torch.as_tensor(ref).numel() == 0:
        return
    rows = row_errors(got, ref)
    worst = int(rows.argmax())
    assert float(rows[worst]) <= TOL[dtype], (f"{what}: row {worst} is off by {float(rows[worst]):.3e} of its own "
                                              f"largest logit, more than {TOL[dtype]:.1e} ({dtype})")
    m = mean_err(got, ref)
    assert m <= MEAN_TOL[dtype], f"{what}: mean error {m:.3e} exceeds {MEAN_TOL[dtype]:.1e} ({dtype})"


def assert_same_engine(a, b, what: str = "", tol: float = 2e-6):
    """Two float32 results of the engine for the same positions, computed in different cuts of the
    work: they differ by the order of a few float32 sums, far less than either differs from
    the float64 plain implementation."""
    e = rel_err(a, b)
    assert e <= tol, f"{what}: the two cuts differ by {e:.3e}, more than {tol:.1e}"


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
