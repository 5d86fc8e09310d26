"""The engine against itself in float32: the same positions computed whole, with the last 32
tokens one by one, and in a batch of unequal lengths must agree far more tightly than any
of them agrees with the float64 plain implementation (each is within 1e-4 of that, so two
could be 2e-4 apart without this check). The cuts differ only in the order of a few float32
sums: products of up to 32 rows sum K per lane and then across lanes, wider ones in chunks
of 16, and a decode step splits a sequence's keys over blocks."""
import pytest
import torch

from conftest import CONFIGS
from helpers import assert_same_engine, tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d"])
def test_three_cuts_agree_in_float32(cuda, model_folders, name):
    import camelid_b200
    from camelid_b200 import StepEntry
    lm = camelid_b200.load(model_folders[name], dtype="float32")
    vocab = CONFIGS[name]["vocab_size"]
    lens = [100, 37, 64, 5]
    seqs = [tokens(600 + i, n, vocab) for i, n in enumerate(lens)]
    cache = lm.new_cache(sum(((n + 63) // 64) * 64 for n in lens) + 128)
    whole = []
    for s in seqs:
        slot = cache.alloc_slot()
        whole.append(lm.step(cache, [StepEntry(slot, s, list(range(len(s))))]).cpu())
        cache.free_slot(slot)
    for s, w in zip(seqs, whole):                       # the prefix in one step, the last 32 one by one
        slot = cache.alloc_slot()
        head = max(1, len(s) - 32)
        got = [lm.step(cache, [StepEntry(slot, s[:head], list(range(head)))]).cpu()]
        got += [lm.step(cache, [StepEntry(slot, [t], [0])]).cpu() for t in s[head:]]
        cache.free_slot(slot)
        assert_same_engine(torch.cat(got), w, f"{name}: {len(s)} tokens whole against prefix + single tokens")
    slots = [cache.alloc_slot() for _ in seqs]          # all four together: half as prompts, then token by token
    half = [max(1, n // 2) for n in lens]
    lg = lm.step(cache, [StepEntry(sl, s[:h], list(range(h))) for sl, s, h in zip(slots, seqs, half)]).cpu()
    off = 0
    for s, h, w in zip(seqs, half, whole):
        assert_same_engine(lg[off:off + h], w[:h], f"{name}: prompt of {h} in a batch against whole")
        off += h
    pos, live = list(half), list(range(len(seqs)))
    while live:
        lg = lm.step(cache, [StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu()
        for r, i in enumerate(live):
            assert_same_engine(lg[r:r + 1], whole[i][pos[i]:pos[i] + 1],
                               f"{name}: request {i} position {pos[i]} in a batch of {len(live)} against whole")
            pos[i] += 1
        for i in [i for i in live if pos[i] >= lens[i]]:
            cache.free_slot(slots[i])
        live = [i for i in live if pos[i] < lens[i]]
    cache.book.audit()
