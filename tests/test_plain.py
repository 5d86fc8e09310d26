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


# ---- the reference's own hand-built models and the numbers its tests expect of them ----

def _select_rows(rows, cols, source_cols, scale=1.0):
    m = torch.zeros(rows, cols)
    for r, c in enumerate(source_cols):
        m[r, c] = scale
    return m


def _session_model():
    """The model of tests/inference_session.rs:545-614: hidden 4, 2 heads on 1 kv head of 2,
    feed-forward 6, vocabulary 3, eps 1e-6, theta 10000; every matrix selects columns. Its
    rotary pairs are adjacent; with a rotary size of 2 that is also the split-half pair."""
    cfg = {"hidden_size": 4, "num_hidden_layers": 1, "intermediate_size": 6, "num_attention_heads": 2,
           "num_key_value_heads": 1, "head_dim": 2, "vocab_size": 3, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
           "tie_word_embeddings": False}
    p = "model.layers.0."
    w = {"model.embed_tokens.weight": torch.tensor([[1.0, 0, 0, 0], [0.5, 0, 0, 0], [0, 1.0, 0, 0]]),
         "model.norm.weight": torch.ones(4),
         "lm_head.weight": torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0], [0, 0, 1.0, 0]]),
         p + "input_layernorm.weight": torch.ones(4), p + "post_attention_layernorm.weight": torch.ones(4),
         p + "self_attn.q_proj.weight": _select_rows(4, 4, [0, 1, 2, 3]),
         p + "self_attn.k_proj.weight": _select_rows(2, 4, [0, 1]),
         p + "self_attn.v_proj.weight": _select_rows(2, 4, [0, 1], 0.5),
         p + "self_attn.o_proj.weight": _select_rows(4, 4, [0, 1, 2, 3]),
         p + "mlp.gate_proj.weight": _select_rows(6, 4, [0, 1, 2, 3, 0, 1]),
         p + "mlp.up_proj.weight": _select_rows(6, 4, [0, 1, 2, 3, 0, 1]),
         p + "mlp.down_proj.weight": _select_rows(4, 6, [0, 1, 2, 3])}
    return cfg, w


def _kept_keys_and_values(cfg, w, ids):
    x = pl.embedding(torch.tensor(ids), w["model.embed_tokens.weight"], torch.float32)
    n = pl.rms_norm(x, w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    _out, (k, v) = pl.attention_block(n, w, "model.layers.0.", cfg, torch.arange(len(ids)), pl.rope_frequencies(cfg))
    return k, v


def test_reference_session_model_keys_and_values_after_one_token():
    """tests/inference_session.rs:27-40: after token 1 the cache holds keys (1.999984, 0) and
    values (0.999992, 0): the norm's scale 1/sqrt(0.25/4 + 1e-6) on 0.5, the value matrix 0.5."""
    cfg, w = _session_model()
    k, v = _kept_keys_and_values(cfg, w, [1])
    assert k.shape == (1, 1, 2) and v.shape == (1, 1, 2)
    assert abs(float(k[0, 0, 0]) - 1.999984) < 5e-4 and abs(float(k[0, 0, 1])) < 5e-4
    assert abs(float(v[0, 0, 0]) - 0.999992) < 5e-4 and abs(float(v[0, 0, 1])) < 5e-4
    logits = pl.forward(cfg, w, [1])
    assert logits.shape == (1, 3) and torch.isfinite(logits).all()


def test_reference_session_model_rotates_the_key_before_it_is_kept():
    """tests/inference_session.rs:43-56: token 2 at position 1 has the key (0, y) before the
    rotation, y = 1/sqrt(0.25 + 1e-6); the cache holds (-y sin 1, y cos 1)."""
    cfg, w = _session_model()
    k, _v = _kept_keys_and_values(cfg, w, [1, 2])
    y = 1.0 / math.sqrt(0.25 + 1e-6)
    assert abs(float(k[1, 0, 0]) + y * math.sin(1.0)) < 5e-4
    assert abs(float(k[1, 0, 1]) - y * math.cos(1.0)) < 5e-4
    assert abs(float(k[0, 0, 0]) - 1.999984) < 5e-4          # the first key is as after one token


def test_reference_session_model_whole_layer_by_hand():
    """The same model carried through the whole layer by hand for token 1 alone (one key: the
    attention output is the value), with the reference's order of operations
    (src/inference.rs:6228-6804): every matrix selects columns, so each step is a line."""
    cfg, w = _session_model()
    s1 = 1.0 / math.sqrt(0.25 / 4 + 1e-6)
    v0 = 0.5 * 0.5 * s1                                   # value = 0.5 * normed x0; both heads copy it
    r = [0.5 + v0, 0.0, v0, 0.0]                          # residual + attention output (heads 0 and 1, first lane each)
    s2 = 1.0 / math.sqrt((r[0] ** 2 + r[2] ** 2) / 4 + 1e-6)
    n2 = [x * s2 for x in r]
    act = [(g / (1 + math.exp(-g))) * g for g in n2]      # gate and up select the same columns
    out = [r[i] + act[i] for i in range(4)]               # down selects the first four of six
    s3 = 1.0 / math.sqrt(sum(x * x for x in out) / 4 + 1e-6)
    want = [out[0] * s3, out[1] * s3, out[2] * s3]        # the output matrix selects columns 0, 1, 2
    got = pl.forward(cfg, w, [1])[0]
    assert torch.allclose(got, torch.tensor(want, dtype=torch.float32), atol=1e-6)


def test_reference_tied_output_rows():
    """src/inference/tests.rs:8830-8852: hidden (2, 3) against the tied embedding rows (1, 0),
    (0, 1), (2, 3) gives logits 2, 3, 13; :8854-8893: (2, -1, 0.5) against the row
    (2, -0.5, 1.5) gives 5.25."""
    cfg = {"tie_word_embeddings": True}
    w = {"model.embed_tokens.weight": torch.tensor([[1.0, 0.0], [0.0, 1.0], [2.0, 3.0]])}
    logits = torch.tensor([[2.0, 3.0]]) @ pl.output_weight(cfg, w).T
    assert torch.allclose(logits, torch.tensor([[2.0, 3.0, 13.0]]), atol=1e-6)
    w = {"model.embed_tokens.weight": torch.tensor([[0.5, 1.0, -2.0], [-1.0, 0.25, 0.75], [2.0, -0.5, 1.5], [0.0, 3.0, -1.0]])}
    logits = torch.tensor([[2.0, -1.0, 0.5]]) @ pl.output_weight(cfg, w).T
    assert abs(float(logits[0, 2]) - 5.25) < 1e-6
    # through forward: an identity layer stack is not available, so the final norm's factor is divided out
    cfg = {"hidden_size": 2, "num_hidden_layers": 0, "num_attention_heads": 1, "head_dim": 2, "vocab_size": 3,
           "rms_norm_eps": 1e-6, "tie_word_embeddings": True}
    w = {"model.embed_tokens.weight": torch.tensor([[1.0, 0.0], [0.0, 1.0], [2.0, 3.0]]), "model.norm.weight": torch.ones(2)}
    got = pl.forward(cfg, w, [2])[0] * math.sqrt((4 + 9) / 2 + 1e-6)
    assert torch.allclose(got, torch.tensor([2.0, 3.0, 13.0]), atol=1e-5)


def test_reference_norm_mean_square():
    """src/inference/tests.rs:1852-1862: (3, 4, 0, -5) has mean square 12.5; the norm's output is
    x / sqrt(12.5 + eps) * weight."""
    x = torch.tensor([[3.0, 4.0, 0.0, -5.0]])
    w = torch.tensor([1.0, 2.0, 3.0, 4.0])
    s = 1 / math.sqrt(12.5 + 1e-5)
    assert torch.allclose(pl.rms_norm(x, w, 1e-5), torch.tensor([[3 * s, 8 * s, 0.0, -20 * s]]), atol=1e-6)
