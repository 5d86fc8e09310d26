"""The engine against the plain implementation, in float32 and in bfloat16: each request
alone and whole; with the last 32 tokens one by one; in batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again; long
decoding; the first tokens of a sequence."""
import pytest
import torch

from conftest import CONFIGS
from helpers import assert_close, oracle, tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]

_models: dict = {}


def load(model_folders, name, dtype):
    import camelid_b200
    key = (name, dtype)
    if key not in _models:
        _models[key] = camelid_b200.load(model_folders[name], dtype=dtype)
    return _models[key]


def run_whole(lm, cache, ids):
    from camelid_b200 import StepEntry
    slot = cache.alloc_slot()
    try:
        return lm.step(cache, [StepEntry(slot, ids, list(range(len(ids))))]).cpu()
    finally:
        cache.free_slot(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,length", [("tiny_a", 1), ("tiny_a", 5), ("tiny_a", 100), ("tiny_b", 2), ("tiny_b", 77),
                                         ("tiny_b", 200), ("tiny_b_odd", 3), ("tiny_b_odd", 130), ("tiny_c", 300), ("tiny_d", 3), ("tiny_d", 300)])
def test_whole_request(cuda, model_folders, name, length, dtype):
    lm = load(model_folders, name, dtype)
    ids = tokens(100 + length, length, CONFIGS[name]["vocab_size"])
    cache = lm.new_cache(512)
    got = run_whole(lm, cache, ids)
    assert_close(got, oracle(model_folders[name], ids), dtype, f"{name} whole {length}")
    cache.book.audit()
    assert cache.book.slots.n_held == 0 and cache.book.pools[0].n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,length", [("tiny_a", 100), ("tiny_b", 150), ("tiny_b_odd", 90), ("tiny_c", 40), ("tiny_d", 170)])
def test_last_32_one_by_one(cuda, model_folders, name, length, dtype):
    """The prefix in one step, then the last 32 tokens (all of them if there are fewer) one
    by one: the same logits as the whole sequence."""
    from camelid_b200 import StepEntry
    lm = load(model_folders, name, dtype)
    ids = tokens(7 + length, length, CONFIGS[name]["vocab_size"])
    ref = oracle(model_folders[name], ids)
    cache = lm.new_cache(256)
    slot = cache.alloc_slot()
    head = max(1, length - 32)
    got = [lm.step(cache, [StepEntry(slot, ids[:head], list(range(head)))]).cpu()]
    for t in range(head, length):
        got.append(lm.step(cache, [StepEntry(slot, [ids[t]], [0])]).cpu())
    cache.free_slot(slot)
    got = torch.cat(got)
    assert_close(got, ref, dtype, f"{name} prefix {head} + {length - head} single tokens")
    first_wrong = None
    for t in range(length):
        if int(got[t].argmax()) != int(ref[t].argmax()):
            top2 = ref[t].topk(2).values
            if float(top2[0] - top2[1]) > 0.05 * float(ref.abs().max()):
                first_wrong = t
                break
    assert first_wrong is None, f"argmax differs first at position {first_wrong} (prefix ends at {head})"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_b_odd", "tiny_d"])
def test_unequal_batches_reuse_slots(cuda, model_folders, name, dtype):
    """Batches of unequal prompts, decoded a different number of steps each so that the
    shorter requests end earlier; three batches one after another in a cache that only fits
    one, so every slot and page is used again."""
    from camelid_b200 import StepEntry
    lm = load(model_folders, name, dtype)
    vocab = CONFIGS[name]["vocab_size"]
    batches = [[(5, 3), (11, 8), (1, 6)], [(17, 2), (2, 12), (40, 5), (9, 1)], [(64, 4), (63, 7), (65, 2)]]
    cache = lm.new_cache(4 * 128, max_slots=4)
    seen_slots = []
    for b, batch in enumerate(batches):
        seqs = [tokens(1000 * b + i, p + d, vocab) for i, (p, d) in enumerate(batch)]
        refs = [oracle(model_folders[name], s) for s in seqs]
        slots = [cache.alloc_slot() for _ in batch]
        seen_slots.append(list(slots))
        live = list(range(len(batch)))
        logits = lm.step(cache, [StepEntry(slots[i], seqs[i][:batch[i][0]], list(range(batch[i][0]))) for i in live]).cpu()
        off = 0
        for i in live:
            p = batch[i][0]
            assert_close(logits[off:off + p], refs[i][:p], dtype, f"{name} batch {b} request {i} prompt")
            off += p
        step = 0
        while live:
            live = [i for i in live if step < batch[i][1]]
            ended = [i for i in range(len(batch)) if slots[i] is not None and i not in live]
            for i in ended:
                cache.free_slot(slots[i])
                slots[i] = None
            if not live:
                break
            logits = lm.step(cache, [StepEntry(slots[i], [seqs[i][batch[i][0] + step]], [0]) for i in live]).cpu()
            for r, i in enumerate(live):
                pos = batch[i][0] + step
                assert_close(logits[r:r + 1], refs[i][pos:pos + 1], dtype,
                             f"{name} batch {b} request {i} decode step {step} (position {pos}, slot {slots[i]})")
            step += 1
        cache.book.audit()
        assert cache.book.slots.n_held == 0 and cache.book.pools[0].n_held == 0
    assert seen_slots[0][0] == seen_slots[1][0] == seen_slots[2][0], "slots were not used again"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_c", "tiny_d"])
def test_long_decoding(cuda, model_folders, name, dtype):
    """A short prompt, then 600 tokens one by one: page boundaries, growing split counts."""
    from camelid_b200 import StepEntry
    lm = load(model_folders, name, dtype)
    ids = tokens(42, 620, CONFIGS[name]["vocab_size"])
    ref = oracle(model_folders[name], ids)
    cache = lm.new_cache(640)
    slot = cache.alloc_slot()
    got = [lm.step(cache, [StepEntry(slot, ids[:20], list(range(20)))]).cpu()]
    for t in range(20, 620):
        got.append(lm.step(cache, [StepEntry(slot, [ids[t]], [0])]).cpu())
    cache.free_slot(slot)
    got = torch.cat(got)
    for lo in range(0, 620, 62):
        assert_close(got[lo:lo + 62], ref[lo:lo + 62], dtype, f"positions {lo}..{lo + 62}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_d"])
def test_first_tokens_one_by_one(cuda, model_folders, name, dtype):
    """A sequence fed one token at a time from its very first token (position 0, the single
    key case), twice in a row in the same slot."""
    from camelid_b200 import StepEntry
    lm = load(model_folders, name, dtype)
    cache = lm.new_cache(64, max_slots=1)
    for rep in range(2):
        ids = tokens(300 + rep, 9, CONFIGS[name]["vocab_size"])
        ref = oracle(model_folders[name], ids)
        slot = cache.alloc_slot()
        assert slot == 0
        got = torch.cat([lm.step(cache, [StepEntry(slot, [t], [0])]).cpu() for t in ids])
        cache.free_slot(slot)
        assert_close(got, ref, dtype, f"{name} token by token, run {rep}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunks_and_want_subsets(cuda, model_folders, dtype):
    """A prompt cut into unequal chunks, logits wanted only at some places, in a batch with
    another request: same logits as whole."""
    from camelid_b200 import StepEntry
    name = "tiny_b"
    lm = load(model_folders, name, dtype)
    vocab = CONFIGS[name]["vocab_size"]
    a, b = tokens(1, 90, vocab), tokens(2, 33, vocab)
    ra, rb = oracle(model_folders[name], a), oracle(model_folders[name], b)
    cache = lm.new_cache(256)
    sa, sb = cache.alloc_slot(), cache.alloc_slot()
    l1 = lm.step(cache, [StepEntry(sa, a[:50], [0, 49]), StepEntry(sb, b[:1], [])]).cpu()
    assert l1.shape[0] == 2
    assert_close(l1, ra[[0, 49]], dtype, "chunk 1")
    l2 = lm.step(cache, [StepEntry(sb, b[1:33], [31]), StepEntry(sa, a[50:90], [39, 0])]).cpu()
    assert_close(l2[0:1], rb[32:33], dtype, "chunk 2, request b")
    assert_close(l2[1:3], ra[[89, 50]], dtype, "chunk 2, request a")
    l3 = lm.step(cache, [StepEntry(sa, [5], [])])
    assert l3.shape == (0, vocab)
    cache.free_slot(sa)
    cache.free_slot(sb)


def test_refused_step_leaves_cache(cuda, model_folders):
    from camelid_b200 import CacheError, StepEntry, StepError
    lm = load(model_folders, "tiny_a", "float32")
    cache = lm.new_cache(128, max_slots=2)
    s = cache.alloc_slot()
    lm.step(cache, [StepEntry(s, [1, 2, 3], [2])])
    before = (cache.length(s), list(cache.book.pages[0][s]), cache.book.pools[0].n_free)
    with pytest.raises(StepError):
        lm.step(cache, [StepEntry(s, [1, 256], [0])])          # id outside the vocabulary
    with pytest.raises(StepError):
        lm.step(cache, [StepEntry(s, [1], [1])])               # wanted place outside the step
    with pytest.raises(StepError):
        lm.step(cache, [StepEntry(s, [], [])])
    with pytest.raises(CacheError):
        lm.step(cache, [StepEntry(s, [1] * 126, [])])          # past the model's 128 positions
    with pytest.raises(CacheError):
        lm.step(cache, [StepEntry(1, [1], [])])                # slot not in use
    assert before == (cache.length(s), list(cache.book.pages[0][s]), cache.book.pools[0].n_free)
    cache.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
def test_more_sequences_than_a_tile_of_rows(cuda, model_folders, name, dtype):
    """140 sequences in one batch: their prompts in one step, then decode steps of 140 rows (more
    than the 128 rows up to which products run transposed), then of 100 after 40 have ended."""
    from camelid_b200 import StepEntry
    lm = load(model_folders, name, dtype)
    vocab = CONFIGS[name]["vocab_size"]
    n, steps = 140, 4
    lens = [1 + (7 * i) % 13 for i in range(n)]
    seqs = [tokens(5000 + i, lens[i] + steps, vocab) for i in range(n)]
    refs = [oracle(model_folders[name], s) for s in seqs]
    cache = lm.new_cache(n * 64, max_slots=n)
    slots = [cache.alloc_slot() for _ in range(n)]
    logits = lm.step(cache, [StepEntry(slots[i], seqs[i][:lens[i]], [lens[i] - 1]) for i in range(n)]).cpu()
    assert_close(logits, torch.stack([refs[i][lens[i] - 1] for i in range(n)]), dtype, f"{name} prompts of {n} sequences")
    live = list(range(n))
    for t in range(steps):
        if t == 2:
            for i in live[100:]:
                cache.free_slot(slots[i])
            live = live[:100]
        logits = lm.step(cache, [StepEntry(slots[i], [seqs[i][lens[i] + t]], [0]) for i in live]).cpu()
        assert_close(logits, torch.stack([refs[i][lens[i] + t] for i in live]), dtype,
                     f"{name} decode step {t} of {len(live)} sequences")
    for i in live:
        cache.free_slot(slots[i])
    cache.book.audit()
    assert cache.book.slots.n_held == 0 and cache.book.pools[0].n_held == 0
