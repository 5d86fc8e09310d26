"""The sizes that bench.py times, against the plain implementation: the Llama 3.2 1B widths
with prompts of lengths uniform in [1, 2048] (one of exactly 2,048) in one prefill step and
decoding at contexts beyond 2,048 positions; the Llama 3.1 8B widths; and the very model the
benchmark draws (16 layers, seed 2, on the device), so that what is timed is what was checked.

The weights are drawn on the device by the library's generator (the host computes the same
numbers: test_random_weights_gpu.py); the plain implementation gets the same tensors and runs
its float64 torch operations on the GPU, where the wide products take seconds instead of
minutes. The wide models have two layers (1B) and one layer (8B): what depends on the
number of layers is covered by the 16-layer run."""
import numpy as np
import pytest
import torch

import plain_llama as pl
from helpers import assert_close, tokens

pytestmark = pytest.mark.gpu


def _build(cfg, seed, dtype):
    """The engine's model and the plain implementation's weights, from one draw on the device."""
    from camelid_b200 import DecoderModel, LanguageModel
    from camelid_b200.weights.random_init import random_tensors
    model = DecoderModel.from_config(cfg, dtype=dtype, device="cuda")
    weights = random_tensors(model.tensor_specs(), seed, torch.bfloat16, "cuda")
    model.load_tensors(weights)
    return LanguageModel(model), weights


def _check(cfg, seed, dtype, lens, decode, chunk=None):
    from camelid_b200 import StepEntry
    lm, weights = _build(cfg, seed, dtype)
    seqs = [tokens(40 + i, n + decode, cfg["vocab_size"]) for i, n in enumerate(lens)]
    want_at = [sorted({0, n // 2, n - 1} | set(range(n, n + decode))) for n in lens]
    cache = lm.new_cache(sum(((len(s) + 63) // 64) * 64 for s in seqs), max_slots=len(seqs))
    slots = [cache.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    lg = lm.step(cache, [StepEntry(sl, s[:n], [a for a in at if a < n]) for sl, s, n, at in zip(slots, seqs, lens, want_at)]).cpu()
    off = 0
    for i, (n, at) in enumerate(zip(lens, want_at)):
        k = len([a for a in at if a < n])
        got[i].append(lg[off:off + k])
        off += k
    for t in range(decode):
        lg = lm.step(cache, [StepEntry(sl, [s[n + t]], [0]) for sl, s, n in zip(slots, seqs, lens)]).cpu()
        for i in range(len(seqs)):
            got[i].append(lg[i:i + 1])
    for sl in slots:
        cache.free_slot(sl)
    lm.model.check_device_errors()
    del lm
    for i, (s, at) in enumerate(zip(seqs, want_at)):
        ref = pl.forward(cfg, weights, s, dtype=torch.float64, rows=at, device="cuda")
        assert_close(torch.cat(got[i]), ref, dtype, f"request {i} ({lens[i]} prompt tokens, places {at})")


def _llama(**over):
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
           "num_hidden_layers": 2, "intermediate_size": 8192, "num_attention_heads": 32, "num_key_value_heads": 8,
           "head_dim": 64, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192}, "tie_word_embeddings": True}
    cfg.update(over)
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_1b_widths_prompts_uniform_up_to_2048(cuda, dtype):
    """Eight prompts, seven of lengths drawn uniformly from [1, 2048] and one of exactly 2,048
    tokens, in one prefill step; then four decode steps of the eight, the longest at positions
    2,048 to 2,051."""
    lens = [int(x) for x in np.random.default_rng(2048).integers(1, 2049, size=7)] + [2048]
    _check(_llama(), 2, dtype, lens, decode=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_8b_widths(cuda, dtype):
    """Hidden 4,096, feed-forward 14,336, heads of 128, an output matrix of its own."""
    cfg = _llama(hidden_size=4096, intermediate_size=14336, head_dim=128, num_hidden_layers=1, tie_word_embeddings=False,
                 rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 8192})
    _check(cfg, 4, dtype, [1500, 37, 2048], decode=3)


def test_the_benchmarks_own_model(cuda):
    """``from_random`` of the benchmark's configuration and seed (all 16 layers, bfloat16): a
    prompt of 256 tokens and two decode steps against the plain implementation, which gets
    the same weights by drawing them again."""
    import camelid_b200
    from camelid_b200 import StepEntry, benchmark
    from camelid_b200.weights.random_init import random_tensors
    cfg = benchmark.config_for(2)
    seed = benchmark.SHAPES[2]["seed"]
    assert cfg["num_hidden_layers"] == 16 and seed == 2
    lm = camelid_b200.from_random(cfg, seed, dtype="bfloat16")
    ids = tokens(77, 258, cfg["vocab_size"])
    cache = lm.new_cache(320, max_slots=1)
    slot = cache.alloc_slot()
    got = [lm.step(cache, [StepEntry(slot, ids[:256], [0, 128, 255])]).cpu()]
    got += [lm.step(cache, [StepEntry(slot, [ids[256 + t]], [0])]).cpu() for t in range(2)]
    lm.model.check_device_errors()
    weights = random_tensors(lm.model.tensor_specs(), seed, torch.bfloat16, "cuda")
    del lm
    ref = pl.forward(cfg, weights, ids, dtype=torch.float64, rows=[0, 128, 255, 256, 257], device="cuda")
    assert_close(torch.cat(got), ref, "bfloat16", "the benchmark's model")
