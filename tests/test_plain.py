"""The plain implementation against closed forms and against expectations that the
reference's own unit tests state (cited at each test)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl


def test_llama3_scaling_closed_form():
    """src/inference/tests.rs:8447-8497: theta 10000, rope_dim 4, factor 8, original 16:
    pair 1 turns by 8 * (10000^-0.5 / 8) at position 8."""
    cfg = {"hidden_size": 4, "num_attention_heads": 1, "head_dim": 4, "rope_theta": 10000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 16}}
    f = pl.rope_frequencies(cfg)
    base = np.float32(10000.0) ** np.float32(-0.5)
    assert abs(f[1] - base / 8) < 1e-9
    smooth = (16 / (2 * math.pi) - 1) / 3         # pair 0: wavelength 2 pi lies between 16/4 and 16/1
    assert abs(float(f[0]) - ((1 - smooth) / 8 + smooth)) < 1e-6
    x = torch.tensor([[[0.0, 0.0, 0.0, 1.0]]])     # split-half: pair 1 is (1, 3)
    y = pl.rope(x, torch.tensor([8]), f)
    ang = 8 * float(base) / 8
    assert torch.allclose(y[0, 0], torch.tensor([0.0, -math.sin(ang), 0.0, math.cos(ang)]), atol=1e-6)
    unscaled = math.sin(8 * float(base))
    assert abs(float(y[0, 0, 1]) + unscaled) > 1e-2


def test_llama3_three_branches():
    cfg = {"hidden_size": 32, "num_attention_heads": 1, "head_dim": 32, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 64}}
    plain = pl.rope_frequencies({**cfg, "rope_scaling": None})
    f = pl.rope_frequencies(cfg)
    wl = 2 * math.pi / plain
    kept, cut, mid = wl < 16, wl > 64, (wl >= 16) & (wl <= 64)
    assert kept.any() and cut.any() and mid.any()
    assert np.array_equal(f[kept], plain[kept])
    assert np.allclose(f[cut], plain[cut] / 4, rtol=1e-6)
    assert ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 4)).all()


def test_rope_rotates_split_half_pairs_and_keeps_norm():
    """Position 1, frequency 1: (x0, x1) -> (x0 cos 1 - x1 sin 1, x0 sin 1 + x1 cos 1), as in
    tests/inference_session.rs:43-56 (key y rotated by sin 1, cos 1)."""
    f = np.array([1.0, 0.0], dtype=np.float32)
    x = torch.tensor([[[0.0, 5.0, 2.0, 7.0]]])
    y = pl.rope(x, torch.tensor([1]), f)[0, 0]
    assert torch.allclose(y, torch.tensor([-2 * math.sin(1.0), 5.0, 2 * math.cos(1.0), 7.0]), atol=1e-6)
    big = torch.randn(6, 3, 8)
    fr = pl.rope_frequencies({"hidden_size": 8, "num_attention_heads": 1, "head_dim": 8})
    assert torch.allclose(pl.rope(big, torch.arange(6), fr).norm(dim=-1), big.norm(dim=-1), atol=1e-5)
    assert torch.equal(pl.rope(big, torch.zeros(6, dtype=torch.long), fr), big)


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = pl.rms_norm(x, w, 1e-5)
    s = 1 / math.sqrt(12.5 + 1e-5)
    assert torch.allclose(y, torch.tensor([[3 * s * 2, 4 * s * 0.5]]), atol=1e-7)


def test_attention_is_causal_grouped_and_scaled():
    torch.manual_seed(0)
    T, nH, nKV, hd = 5, 4, 2, 8
    q, k, v = torch.randn(T, nH, hd), torch.randn(T, nKV, hd), torch.randn(T, nKV, hd)
    out = pl.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # one key: a copy of v
    h, t = 2, 3                                                                           # head 2 reads kv head 1
    s = torch.tensor([float(q[t, h] @ k[j, 1]) / math.sqrt(hd) for j in range(t + 1)])
    p = torch.softmax(s, 0)
    assert torch.allclose(out[t, h], (p[:, None] * v[:t + 1, 1]).sum(0), atol=1e-6)
    k2, v2 = k.clone(), v.clone()
    k2[4], v2[4] = 100.0, 100.0
    assert torch.allclose(pl.attention(q, k2, v2)[:4], out[:4])                          # the future is not seen
    w = pl.attention(q, k, v, window=2)
    s = torch.tensor([float(q[t, h] @ k[j, 1]) / math.sqrt(hd) for j in (2, 3)])
    p = torch.softmax(s, 0)
    assert torch.allclose(w[t, h], p[0] * v[2, 1] + p[1] * v[3, 1], atol=1e-6)


def test_swiglu_formula():
    x = torch.tensor([[1.0, -2.0]])
    wg, wu, wd = torch.tensor([[0.5, 0.25]]), torch.tensor([[1.0, 1.0]]), torch.tensor([[2.0], [3.0]])
    g, u = 0.5 - 0.5, 1.0 - 2.0
    act = (g / (1 + math.exp(-g))) * u
    assert torch.allclose(pl.swiglu(x, wg, wu, wd), torch.tensor([[2 * act, 3 * act]]))
    x = torch.tensor([[2.0, 0.0]])
    g, u = 1.0, 2.0
    act = (g / (1 + math.exp(-g))) * u
    assert torch.allclose(pl.swiglu(x, wg, wu, wd), torch.tensor([[2 * act, 3 * act]]))


def test_forward_is_causal_and_tied_output(model_folders):
    cfg, w = pl.read_model(model_folders["tiny_a"])
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    full = pl.forward(cfg, w, ids)
    assert full.shape == (8, 256)
    assert torch.allclose(pl.forward(cfg, w, ids[:5]), full[:5], atol=1e-5)
    assert "lm_head.weight" not in w and pl.output_weight(cfg, w) is w["model.embed_tokens.weight"]
    cfg_b, w_b = pl.read_model(model_folders["tiny_b"])
    assert pl.output_weight(cfg_b, w_b) is w_b["lm_head.weight"]
    with pytest.raises(ValueError):
        pl.forward(cfg, w, [256])
    f64 = pl.forward(cfg, w, ids, dtype=torch.float64)
    assert float((f64 - full.double()).abs().max()) < 1e-5
    twice = pl.forward(cfg, w, ids, schedule=[(0, None), (1, None), (0, None), (1, 1)])
    assert not torch.allclose(twice, full)


def test_greedy_ties_and_errors():
    """tests/inference_session.rs:148-154: [0.5, 2.0, 2.0, -1.0] -> 1."""
    assert pl.greedy(np.array([0.5, 2.0, 2.0, -1.0], dtype=np.float32)) == 1
    with pytest.raises(ValueError):
        pl.greedy(np.array([0.0, np.nan], dtype=np.float32))
    assert pl.sample(np.array([0.5, 2.0, 2.0, -1.0], dtype=np.float32), [], temperature=0.0, top_k=2, top_p=0.5, seed=42) == 1


def test_sampler_matches_the_reference_expectations():
    """tests/inference_session.rs:172-198 (top_k 1 -> 0; top_p 0.8 with seed 0 -> 1),
    :216-240 (bias, penalties), :259-293 (top_k 1 and min_p 1 for any seed)."""
    l3 = np.array([3.0, 2.0, 1.0], dtype=np.float32)
    assert pl.sample(l3, [], temperature=1.0, top_k=1, seed=0) == 0
    assert pl.sample(l3, [], temperature=1.0, top_p=0.8, seed=0) == 1
    assert pl.sample(np.array([0.0, 0.5, 0.4], dtype=np.float32), [], logit_bias=[(2, 0.2)]) == 2
    assert pl.sample(np.array([1.0, 0.9, 0.0], dtype=np.float32), [0, 0], presence_penalty=0.5, frequency_penalty=0.25) == 1
    for seed in (0, 1, 7, 42, 123456789):
        assert pl.sample(l3, [], temperature=1.0, top_k=1, seed=seed) == 0
        assert pl.sample(l3, [], temperature=1.0, min_p=1.0, seed=seed) == 0
    l4 = np.array([1.0, 0.5, 0.25, 0.0], dtype=np.float32)
    for seed in (0, 3, 17, 555):
        assert pl.sample(l4, [], temperature=1.0, seed=seed) == pl.sample(l4, [], temperature=1.0, min_p=0.0, seed=seed)
    with pytest.raises(ValueError):
        pl.sample(np.array([0.0, 1.0], dtype=np.float32), [], logit_bias=[(2, 1.0)])


def test_draws_are_a_stream_over_positions():
    d = [pl.unit_draw(7, p) for p in range(200)]
    assert all(0.0 <= x < 1.0 for x in d) and len(set(d)) > 190
    assert abs(float(np.mean(d)) - 0.5) < 0.08
    assert pl.unit_draw(7, 3) == pl.unit_draw(7, 3) != pl.unit_draw(8, 3)
    assert pl.splitmix64(0) == 0 and pl.splitmix64(1) == 0x5692161D100B05E5


def test_sampling_frequencies_follow_the_softmax():
    logits = np.array([2.0, 1.0, 0.0, -1.0], dtype=np.float32)
    counts = np.zeros(4)
    for pos in range(4000):
        counts[pl.sample(logits, [0] * pos, temperature=1.0, seed=11)] += 1
    p = np.exp(logits) / np.exp(logits).sum()
    assert np.abs(counts / 4000 - p).max() < 0.03


def test_generate_stops_and_keeps_the_stop_token(model_folders):
    cfg, w = pl.read_model(model_folders["tiny_b"])
    free = pl.generate(cfg, w, [[5, 6, 7]], 6)[0]
    assert len(free) == 6
    stopped = pl.generate(cfg, w, [[5, 6, 7]], 6, stop_ids=(free[2],))[0]
    assert stopped == free[:free.index(free[2]) + 1]


def test_pinned_logits_of_the_micro_model():
    """tests/golden/plain_micro.json was written by tests/golden/make_golden.py from weights of
    a generator written out there; the plain implementation must still give those logits."""
    import importlib.util
    import json
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(os.path.join(here, "golden", "plain_micro.json")) as f:
        want = json.load(f)
    got = mod.compute()
    assert got["argmax_per_position"] == want["argmax_per_position"]
    assert np.allclose(got["logits_last"], want["logits_last"], atol=1e-9)
    assert np.allclose(got["logits_first"], want["logits_first"], atol=1e-9)
    assert abs(got["sum_abs"] - want["sum_abs"]) < 1e-6
