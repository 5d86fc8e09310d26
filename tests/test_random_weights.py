"""The library's random weights: the host's vectorised generator against the plain
implementation's element-at-a-time restatement, the distribution it draws from, and that a
tensor depends on its own name and the seed only. (Host against device: test_random_weights_gpu.py.)"""
import math

import numpy as np
import torch

import plain_llama as pl
from camelid_b200.parts.base import TensorSpec
from camelid_b200.weights import counter_random as cr
from camelid_b200.weights.random_init import random_slice, random_tensor, random_tensors


def test_host_generator_equals_the_plain_restatement_bit_for_bit():
    for seed, name, kind in ((0, "model.embed_tokens.weight", "linear"), (2, "model.layers.7.mlp.down_proj.weight", "linear"),
                             (2**63 + 5, "model.norm.weight", "norm")):
        for first in (0, 1, 12345, 2**31 - 3, 2**33 + 7):
            got = random_slice(name, kind, seed, first, 64).numpy()
            want = np.array([pl.random_weight(seed, name, first + i, kind) for i in range(64)], dtype=np.float32)
            assert got.tobytes() == want.tobytes(), (seed, name, first)


def test_every_branch_of_the_generator_is_met():
    """All eight octants of the angle, both mantissa ranges of the logarithm, u1 = 1 (radius 0)."""
    key = cr.tensor_key(3, "x")
    z = cr.standard_normals(key, 0, 200000)
    assert np.isfinite(z).all()
    with np.errstate(over="ignore"):
        bits = cr._splitmix64_np(np.uint64(key) + np.arange(1, 200001, dtype=np.uint64) * np.uint64(cr.GOLDEN))
    assert set(((bits & np.uint64(0xFFFFFFFF)) >> np.uint64(29)).tolist()) == set(range(8))
    mant, _ = np.frexp((bits >> np.uint64(32)).astype(np.float64) + 1.0)
    assert (mant < cr.SQRT_HALF).any() and (mant >= cr.SQRT_HALF).any()


def test_polynomials_are_the_functions():
    rng = np.random.default_rng(0)
    t = rng.uniform(0, cr.PI_4, 1000)
    assert np.abs(cr._horner(cr.COS_TERMS, t * t) - np.cos(t)).max() < 2e-16
    assert np.abs(t * cr._horner(cr.SIN_TERMS, t * t) - np.sin(t)).max() < 2e-16
    m = rng.uniform(cr.SQRT_HALF, 2 * cr.SQRT_HALF, 1000)
    s = (m - 1) / (m + 1)
    assert np.abs(2 * s * cr._horner(cr.LOG_TERMS, s * s) - np.log(m)).max() < 2e-16


def test_distribution_is_normal():
    x = cr.standard_normals(cr.tensor_key(11, "some.weight"), 0, 1 << 20)
    n = x.size
    assert abs(x.mean()) < 4 / math.sqrt(n)
    assert abs(x.var() - 1) < 4 * math.sqrt(2 / n)
    assert abs((x ** 3).mean()) < 4 * math.sqrt(15 / n)
    assert abs((x ** 4).mean() - 3) < 4 * math.sqrt(96 / n)
    # Kolmogorov-Smirnov against the normal distribution function
    xs = np.sort(x)
    cdf = 0.5 * (1 + np.array([math.erf(v / math.sqrt(2)) for v in xs[::64]]))
    emp = (np.arange(n)[::64] + 0.5) / n
    assert np.abs(cdf - emp).max() < 1.95 / math.sqrt(n) + 64 / n
    # neighbours in the counter are not correlated
    assert abs(np.mean(x[:-1] * x[1:])) < 4 / math.sqrt(n)
    assert x.max() > 4.0 and x.min() < -4.0


def test_a_tensor_depends_on_its_name_and_the_seed_only():
    spec = TensorSpec((5, 8), "linear")
    a = random_tensor("a.weight", spec, 4, torch.float32)
    both = random_tensors({"b.weight": TensorSpec((3, 3)), "a.weight": spec}, 4, torch.float32)
    assert torch.equal(a, both["a.weight"])
    assert not torch.equal(a, random_tensor("a.weight", spec, 5, torch.float32))
    assert not torch.equal(a, random_tensor("c.weight", spec, 4, torch.float32))
    # a slice is the tensor's elements in row-major order; bfloat16 rounds the float32 draw
    assert torch.equal(random_slice("a.weight", "linear", 4, 8, 16), a.reshape(-1)[8:24])
    assert torch.equal(random_tensor("a.weight", spec, 4, torch.bfloat16), a.to(torch.bfloat16))
    norm = random_tensor("n.weight", TensorSpec((4096,), "norm"), 4, torch.float32)
    assert abs(float(norm.mean()) - 1.0) < 2e-3 and abs(float(norm.std()) - 0.02) < 2e-3
    assert abs(float(random_tensor("w", TensorSpec((64, 64)), 4, torch.float32).std()) - 0.02) < 2e-3
