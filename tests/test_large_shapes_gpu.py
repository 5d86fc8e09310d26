"""The benchmark's widths (Llama 3.2 1B: hidden 2048, 32/8 heads of 64, feed-forward 8192,
vocabulary 128256, llama3 scaling with factor 32) with two layers, so that the kernels run
at the tile counts, split counts and strides of the real model: float32 against the plain
implementation, bfloat16 against it too, unequal prompts, then decoding; and the widths of
the 3B shape (head size 128, 24/8 heads) in one layer."""
import pytest
import torch

import plain_llama as pl
from helpers import assert_close, tokens

pytestmark = pytest.mark.gpu


def _folder(tmp_path_factory, name, **over):
    from camelid_b200.weights.random_init import write_random_model
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
           "num_hidden_layers": 2, "intermediate_size": 8192, "num_attention_heads": 32, "num_key_value_heads": 8,
           "head_dim": 64, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192}, "tie_word_embeddings": True, **over}
    d = str(tmp_path_factory.mktemp(name))
    write_random_model(d, cfg, 2, torch.bfloat16, device="cuda")
    return d, cfg


@pytest.fixture(scope="module")
def shape_1b(tmp_path_factory):
    return _folder(tmp_path_factory, "shape1b")


@pytest.fixture(scope="module")
def shape_3b(tmp_path_factory):
    return _folder(tmp_path_factory, "shape3b", hidden_size=3072, num_attention_heads=24, head_dim=128,
                   num_hidden_layers=1, vocab_size=32000)


def _check(folder, cfg, dtype, lens, decode, options=None):
    import camelid_b200
    from camelid_b200 import StepEntry
    lm = camelid_b200.load(folder, dtype=dtype, options=options)
    config, w = pl.read_model(folder)
    seqs = [tokens(40 + i, n + decode, cfg["vocab_size"]) for i, n in enumerate(lens)]
    # the oracle's logits only at the places that are compared (its output product is the slow part)
    want_at = [sorted({0, n // 2, n - 1} | set(range(n, n + decode))) for n in lens]
    refs = []
    for s, at in zip(seqs, want_at):
        refs.append(pl.forward({**config}, w, s, dtype=torch.float64, rows=at))
    cache = lm.new_cache(sum(((len(s) + 63) // 64) * 64 for s in seqs))
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
    for i in range(len(seqs)):
        assert_close(torch.cat(got[i]), refs[i], dtype, f"request {i} ({lens[i]} prompt tokens)")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_1b_widths_unequal_prompts_then_decode(cuda, shape_1b, dtype):
    folder, cfg = shape_1b
    _check(folder, cfg, dtype, lens=[130, 7, 300, 64], decode=3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_3b_widths_head_size_128(cuda, shape_3b, dtype):
    folder, cfg = shape_3b
    _check(folder, cfg, dtype, lens=[200, 65], decode=2)


def test_norm_inside_the_product_before_it_or_on_its_own(cuda, shape_1b):
    """A prefill of many rows runs each norm inside the products around it (the one before adds
    into the residual stream and writes the rows times the norm's weight, the one after applies
    the rows' scale); with that switched off the norm is a kernel of its own. Both match the
    plain implementation, and a launch count shows that the switch does switch. (Enough rows that
    the narrow products have tiles for most SMs: with fewer they split K and leave their sums to
    the norm kernel, as decode steps do.)"""
    from camelid_b200 import KernelOptions
    from camelid_b200.csrc import ops
    folder, cfg = shape_1b
    counts = []
    for fuse in (True, False):
        before = ops.launch_count()
        _check(folder, cfg, "bfloat16", lens=[900, 400], decode=1, options=KernelOptions(fuse_norm=fuse))
        counts.append(ops.launch_count() - before)
    assert counts[0] < counts[1]
