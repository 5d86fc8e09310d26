"""The device sampler against the plain sampler, fed the same logits."""
import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu


def _sample(cuda, logits, histories, **opts):
    from camelid_b200.sampling import Sampler, SamplingOptions
    s = Sampler(SamplingOptions(**opts), logits.shape[1], cuda)
    out = s.sample(torch.tensor(logits, dtype=torch.float32, device=cuda), histories)
    s.check()
    return out.cpu().tolist()


def test_greedy_ties_and_many_rows(cuda):
    rng = np.random.default_rng(0)
    logits = rng.normal(size=(9, 5003)).astype(np.float32)
    logits[2, 77] = logits[2, 4000] = 9.0            # equal maxima: the lower index wins
    logits[5, :] = 1.0
    got = _sample(cuda, logits, [[]] * 9)
    assert got == [pl.greedy(r) for r in logits] and got[2] == 77 and got[5] == 0
    assert _sample(cuda, np.array([[0.5, 2.0, 2.0, -1.0]], dtype=np.float32), [[]]) == [1]


def test_non_finite_logits_are_an_error(cuda):
    from camelid_b200 import SamplingError
    bad = np.zeros((2, 300), dtype=np.float32)
    bad[1, 5] = np.nan
    with pytest.raises(SamplingError):
        _sample(cuda, bad, [[], []])
    with pytest.raises(SamplingError):
        _sample(cuda, bad, [[], []], temperature=1.0)


@pytest.mark.parametrize("opts", [
    dict(temperature=1.0), dict(temperature=0.7, seed=3), dict(temperature=1.5, top_k=5, seed=1),
    dict(temperature=1.0, top_p=0.8, seed=0), dict(temperature=1.0, min_p=0.1, seed=9),
    dict(temperature=0.9, top_k=50, top_p=0.9, min_p=0.02, seed=123456789),
    dict(temperature=1.0, top_k=1, seed=7), dict(temperature=1.0, min_p=1.0, seed=5),
    dict(temperature=2.0, top_k=1000000, seed=2),
])
def test_stochastic_sampler_matches_plain(cuda, opts):
    rng = np.random.default_rng(42)
    vocab = 1531
    logits = (rng.normal(size=(40, vocab)) * 2.5).astype(np.float32)
    logits[3, 10] = logits[3, 900] = logits[3].max() + 1.0          # ties at the top
    histories = [[1] * (r % 13) for r in range(40)]                 # different stream positions
    got = _sample(cuda, logits, histories, **opts)
    want = [pl.sample(logits[r], histories[r], **opts) for r in range(40)]
    assert got == want


def test_reference_expectations_on_the_device(cuda):
    """tests/inference_session.rs:172-198, :216-240."""
    l3 = np.array([[3.0, 2.0, 1.0]], dtype=np.float32)
    assert _sample(cuda, l3, [[]], temperature=1.0, top_k=1, seed=0) == [0]
    assert _sample(cuda, l3, [[]], temperature=1.0, top_p=0.8, seed=0) == [1]
    assert _sample(cuda, np.array([[0.0, 0.5, 0.4]], dtype=np.float32), [[]], logit_bias=[(2, 0.2)]) == [2]
    assert _sample(cuda, np.array([[1.0, 0.9, 0.0]], dtype=np.float32), [[0, 0]], presence_penalty=0.5,
                   frequency_penalty=0.25) == [1]


def test_adjustments_match_plain(cuda):
    rng = np.random.default_rng(5)
    logits = rng.normal(size=(6, 400)).astype(np.float32)
    histories = [[int(x) for x in rng.integers(0, 400, size=20 + r)] for r in range(6)]
    opts = dict(temperature=0.8, seed=4, repeat_penalty=1.3, presence_penalty=0.4, frequency_penalty=0.2,
                logit_bias=[(7, 5.0), (8, -3.0)])
    got = _sample(cuda, logits, histories, **opts)
    assert got == [pl.sample(logits[r], histories[r], **opts) for r in range(6)]
    from camelid_b200.sampling import Sampler, SamplingOptions
    s = Sampler(SamplingOptions(**opts), 400, cuda)
    dev = torch.tensor(logits, device=cuda)
    s.sample(dev, histories)
    adj = {k: v for k, v in opts.items() if k not in ("temperature", "seed")}
    want = np.stack([pl.adjust_logits(logits[r], histories[r], **adj) for r in range(6)])
    assert np.allclose(dev.cpu().numpy(), want, atol=1e-6)


def test_large_vocabulary_frequencies(cuda):
    """At the real vocabulary size the draws follow the softmax (a few heavy tokens)."""
    vocab = 128256
    logits = np.full((1, vocab), -20.0, dtype=np.float32)
    logits[0, [5, 70000, 128255]] = [2.0, 1.0, 0.0]
    p = np.exp([2.0, 1.0, 0.0]) / np.exp([2.0, 1.0, 0.0]).sum()
    rows = np.repeat(logits, 64, axis=0)
    counts = {5: 0, 70000: 0, 128255: 0}
    for rep in range(8):
        got = _sample(cuda, rows, [[0] * (rep * 64 + r) for r in range(64)], temperature=1.0, seed=11)
        for t in got:
            counts[t] = counts.get(t, 0) + 1
    freq = np.array([counts[5], counts[70000], counts[128255]]) / 512
    assert np.abs(freq - p).max() < 0.07 and sum(counts.values()) == 512


def _seed_with_draw(lo, hi, position):
    """A seed whose draw at ``position`` lies in [lo, hi)."""
    for seed in range(1, 200000):
        if lo <= float(pl.unit_draw(seed, position)) < hi:
            return seed
    raise AssertionError("no seed found")


def _interval_of(row, token, temperature, top_k=None, top_p=None, min_p=None):
    """The stretch of the cumulative distribution that belongs to ``token`` when the sampler's steps
    (src/inference.rs:5991-6091) are done in float64: candidates by logit descending and index ascending, top_k,
    softmax of logit / T, min_p, top_p prefix, each renormalised. None if the token is no candidate."""
    v = row.astype(np.float64)
    order = np.lexsort((np.arange(v.shape[0]), np.signbit(row), -v))       # the reference's total order: +0.0 before -0.0
    if top_k is not None:
        order = order[:min(top_k, order.shape[0])]
    w = np.exp((v[order] - v[order].max()) / temperature)
    prob = w / w.sum()
    if min_p is not None and min_p > 0.0:
        keep = prob >= min_p * prob.max()
        order, prob = order[keep], prob[keep] / prob[keep].sum()
    if top_p is not None and top_p < 1.0:
        n = int(np.searchsorted(np.cumsum(prob), top_p, side="left")) + 1
        order, prob = order[:n], prob[:n] / prob[:n].sum()
    where = np.nonzero(order == token)[0]
    if where.size == 0:
        return None
    cum = np.cumsum(prob)
    i = int(where[0])
    return float(cum[i] - prob[i]), float(cum[i]) if i + 1 < order.shape[0] else 2.0


@pytest.mark.parametrize("case", ["top", "tail", "cold top-k", "nucleus", "all filters", "ties"])
def test_sampler_at_a_large_vocabulary(cuda, case):
    """The two-pass selection at a vocabulary of 50,000: the draw must lie in the chosen token's own stretch of
    the cumulative distribution, computed in float64 (the plain sampler adds 50,000 float32 terms one by one
    and drifts by more than a token's width out in the tail, so token-for-token equality is asked only at the
    small vocabulary above). Draws that land among the few heavy tokens and far out in the crowded tail (where
    a bin holds more keys than the kernel's list and is divided), a low temperature with top-k (the k-th value
    lies beyond the binned range), and thousands of equal logits with the draw among them (equal values are
    ordered by index: the digit-by-digit selection takes over; a token's stretch there is 3e-5 wide, the
    slack 2e-6)."""
    rng = np.random.default_rng(7)
    vocab = 50000
    logits = (rng.normal(size=(4, vocab)) * 2.5).astype(np.float32)
    logits[1] *= 2.5
    if case == "top":
        opts, want_draw = dict(temperature=0.8), (0.0, 0.001)
    elif case == "tail":
        opts, want_draw = dict(temperature=30.0), (0.9995, 1.0)
    elif case == "cold top-k":
        opts, want_draw = dict(temperature=0.05, top_k=300), (0.5, 0.6)
    elif case == "nucleus":
        opts, want_draw = dict(temperature=1.0, top_p=0.95), (0.93, 0.97)
    elif case == "all filters":
        opts, want_draw = dict(temperature=1.2, top_k=1000, top_p=0.9, min_p=0.001), (0.0, 1.0)
    else:
        logits[:, 100:30000] = 1.5                     # 29,900 equal values above most of the rest
        opts, want_draw = dict(temperature=2.0), (0.4, 0.6)
    seed = _seed_with_draw(*want_draw, 0)
    got = _sample(cuda, logits, [[]] * 4, seed=seed, **opts)
    draw = float(pl.unit_draw(seed, 0))
    for r in range(4):
        span = _interval_of(logits[r], got[r], **opts)
        assert span is not None, (r, got[r], "not a candidate")
        assert span[0] - 2e-6 <= draw < span[1] + 2e-6, (r, got[r], span, draw)
