"""Schedules of the engine beyond the everyday ones: decoding past 8,192 positions (where a
sequence's keys are split over more blocks than a cluster has and the attention runs as rotary
kernel + ticket-merged kernel), more query heads per kv head than the fused decode kernel
takes, rolling a slot back (``truncate``) and going on with other tokens, and greedy
generation with the token fed back on the device."""
import pytest
import torch

import plain_llama as pl
from conftest import CONFIGS, TINY_D
from helpers import assert_close, oracle, tokens

pytestmark = pytest.mark.gpu


def _long_model(tmp_path_factory, name, **over):
    from camelid_b200.weights.random_init import write_random_model
    cfg = {**TINY_D, "max_position_embeddings": 12288, **over}
    d = str(tmp_path_factory.mktemp(name))
    write_random_model(d, cfg, 13, torch.bfloat16)
    return d, cfg


@pytest.fixture(scope="module")
def long_d(tmp_path_factory):
    return _long_model(tmp_path_factory, "long_d")


@pytest.fixture(scope="module")
def many_heads(tmp_path_factory):
    return _long_model(tmp_path_factory, "many_heads", hidden_size=272, num_attention_heads=34, num_key_value_heads=1,
                       max_position_embeddings=2048)


def _prefill_then_decode(folder, cfg, dtype, n_prompt, n_decode, chunk, seen: dict | None = None):
    import camelid_b200
    from camelid_b200 import StepEntry
    from camelid_b200.csrc import ops
    lm = camelid_b200.load(folder, dtype=dtype)
    ids = tokens(8, n_prompt + n_decode, cfg["vocab_size"])
    want = sorted({0, n_prompt // 2, n_prompt - 1} | set(range(n_prompt, n_prompt + n_decode)))
    cfg_p, w = pl.read_model(folder)
    ref = pl.forward(cfg_p, w, ids, dtype=torch.float64, rows=want, device="cuda")
    cache = lm.new_cache(((len(ids) + 63) // 64) * 64, max_slots=1)
    slot = cache.alloc_slot()
    got = []
    for lo in range(0, n_prompt, chunk):
        hi = min(lo + chunk, n_prompt)
        at = [a - lo for a in want if lo <= a < hi]
        got.append(lm.step(cache, [StepEntry(slot, ids[lo:hi], at)]).cpu())
    if seen is not None:                  # which attention kernels the decode steps launch
        for name in ("rope_kv_from_partials", "attn_paged_mma", "attn_decode_fused"):
            real = getattr(ops, name)

            def counting(*a, _real=real, _name=name, **k):
                seen[_name] = seen.get(_name, 0) + 1
                return _real(*a, **k)
            setattr(ops, name, counting)
    try:
        for t in range(n_prompt, n_prompt + n_decode):
            got.append(lm.step(cache, [StepEntry(slot, [ids[t]], [0])]).cpu())
    finally:
        if seen is not None:
            for name in ("rope_kv_from_partials", "attn_paged_mma", "attn_decode_fused"):
                setattr(ops, name, getattr(ops, name).__kwdefaults__["_real"])
    cache.free_slot(slot)
    lm.model.check_device_errors()
    assert_close(torch.cat(got), ref, dtype, f"{n_prompt} prompt tokens in chunks of {chunk}, then {n_decode} single tokens")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_decoding_past_8192_positions(cuda, long_d, dtype):
    """A prompt of 8,300 tokens in chunks, then 40 tokens one by one through the captured
    graph: in bfloat16 the keys of the one sequence want 33 blocks per kv head, more than a
    cluster, so the steps run the rotary kernel on the product's split sums and the attention
    kernel whose last block merges the splits."""
    folder, cfg = long_d
    seen = {}
    _prefill_then_decode(folder, cfg, dtype, 8300, 40, 2048, seen)
    if dtype == "bfloat16":
        assert seen.get("rope_kv_from_partials", 0) > 0 and seen.get("attn_paged_mma", 0) > 0, seen
        assert seen.get("attn_decode_fused", 0) == 0, seen


def test_more_query_heads_per_kv_head_than_the_fused_kernel_takes(cuda, many_heads):
    """34 query heads on one kv head of 64: bfloat16 decode steps leave the fused kernel for the
    rotary kernel and the attention kernel with three chunks of heads."""
    folder, cfg = many_heads
    seen = {}
    _prefill_then_decode(folder, cfg, "bfloat16", 700, 12, 512, seen)
    assert seen.get("attn_paged_mma", 0) > 0 and seen.get("attn_decode_fused", 0) == 0, seen


@pytest.mark.parametrize("how", ["one step", "token by token"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
def test_truncate_then_other_tokens(cuda, model_folders, name, dtype, how):
    """A prompt of 100 tokens, 10 single tokens, the slot rolled back to 70 positions, then 20
    other tokens (in one step, or one by one through the captured graph, whose block tables
    must notice the roll-back): the logits are those of the spliced sequence."""
    import camelid_b200
    from camelid_b200 import StepEntry
    lm = camelid_b200.load(model_folders[name], dtype=dtype)
    vocab = CONFIGS[name]["vocab_size"]
    first, other = tokens(1, 110, vocab), tokens(2, 20, vocab)
    cache = lm.new_cache(256, max_slots=2)
    keep = cache.alloc_slot()                                    # a neighbour that must stay as it is
    neighbour = tokens(3, 40, vocab)
    lm.step(cache, [StepEntry(keep, neighbour[:39], [])])
    slot = cache.alloc_slot()
    lm.step(cache, [StepEntry(slot, first[:100], [99])])
    for t in range(100, 110):
        lm.step(cache, [StepEntry(slot, [first[t]], [0])])
    assert cache.length(slot) == 110
    cache.truncate(slot, 70)
    assert cache.length(slot) == 70
    spliced = first[:70] + other
    ref = oracle(model_folders[name], spliced)
    if how == "one step":
        got = lm.step(cache, [StepEntry(slot, other, list(range(20)))]).cpu()
    else:
        got = torch.cat([lm.step(cache, [StepEntry(slot, [t], [0])]).cpu() for t in other])
    assert_close(got, ref[70:], dtype, f"{name}: 20 tokens after a roll-back to 70")
    last = lm.step(cache, [StepEntry(keep, [neighbour[39]], [0])]).cpu()
    assert_close(last, oracle(model_folders[name], neighbour)[39:], dtype, f"{name}: the neighbouring slot")
    cache.free_slot(slot)
    cache.free_slot(keep)
    cache.book.audit()


def test_greedy_generation_fed_on_the_device(cuda, model_folders):
    """Greedy requests decode with the token fed back inside the captured step. float32, tiny_a:
    token for token the plain loop, with and without stop tokens, and the same tokens as the
    loop that reads every token back before the next step. bfloat16, tiny_d: every token is a
    best token of the plain implementation given the tokens before it."""
    import camelid_b200
    from camelid_b200 import KernelOptions
    name = "tiny_a"
    cfg, w = pl.read_model(model_folders[name])
    prompts = [tokens(50 + i, n, CONFIGS[name]["vocab_size"]) for i, n in enumerate([5, 11, 1])]
    want = pl.generate(cfg, w, prompts, 40, dtype=torch.float64)
    fed = camelid_b200.load(model_folders[name], dtype="float32")
    fed_runs = []
    real = fed.model.decode_fed
    fed.model.decode_fed = lambda *a, **k: (fed_runs.append(a[3]), real(*a, **k))[1]
    assert fed.generate(prompts, max_tokens=40, stop_token_ids=()) == want
    assert fed_runs == [39]
    stop = want[1][20]
    want_stop = pl.generate(cfg, w, prompts, 40, stop_ids=(stop,), dtype=torch.float64)
    assert fed.generate(prompts, max_tokens=40, stop_token_ids=(stop,)) == want_stop
    assert any(len(x) < 40 for x in want_stop)
    unfed = camelid_b200.load(model_folders[name], dtype="float32", options=KernelOptions(feed_on_device=False))
    assert unfed.generate(prompts, max_tokens=40, stop_token_ids=()) == want
    name = "tiny_d"
    cfg, w = pl.read_model(model_folders[name])
    lm = camelid_b200.load(model_folders[name], dtype="bfloat16")
    prompts = [tokens(70 + i, n, CONFIGS[name]["vocab_size"]) for i, n in enumerate([30, 3])]
    got = lm.generate(prompts, max_tokens=70, stop_token_ids=())
    for p, g in zip(prompts, got):
        assert len(g) == 70
        ref = pl.forward(cfg, w, (p + g)[:-1], dtype=torch.float64)
        scale = float(ref.abs().max())
        for i, tok in enumerate(g):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 3e-2 * scale, f"token {i} of request with {len(p)} prompt tokens"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
def test_a_layout_seen_again_replays_a_captured_step(cuda, model_folders, name, dtype):
    """Steps of several tokens per sequence whose layout (tokens per sequence, wanted places, block
    table widths) comes back run as a captured graph from the second time on: other tokens, other
    slots and other starting positions must give their own logits, and a different layout in
    between must not disturb them."""
    import camelid_b200
    from camelid_b200 import StepEntry
    lm = camelid_b200.load(model_folders[name], dtype=dtype)
    assert lm.model.capture_steps
    vocab = CONFIGS[name]["vocab_size"]
    cache = lm.new_cache(1024, max_slots=6)
    lens = [37, 5, 64]
    for rep in range(4):
        if rep == 2:                                   # another layout in between, and a shift of the slots
            extra = cache.alloc_slot()
            ids = tokens(900, 21, vocab)
            got = lm.step(cache, [StepEntry(extra, ids, [20])]).cpu()
            assert_close(got, oracle(model_folders[name], ids)[20:], dtype, "the layout in between")
        seqs = [tokens(700 + 10 * rep + i, n + 9, vocab) for i, n in enumerate(lens)]
        slots = [cache.alloc_slot() for _ in seqs]
        # a first chunk of 9 tokens each (its own layout), then the layout under test on top of it
        lm.step(cache, [StepEntry(s, q[:9], []) for s, q in zip(slots, seqs)])
        got = lm.step(cache, [StepEntry(s, q[9:], [0, len(q) - 10]) for s, q in zip(slots, seqs)]).cpu()
        for i, q in enumerate(seqs):
            ref = oracle(model_folders[name], q)
            assert_close(got[2 * i:2 * i + 2], ref[[9, len(q) - 1]], dtype, f"{name} round {rep} request {i}")
        for s in slots:
            cache.free_slot(s)
    graphs = lm.model._step_graphs[cache]
    assert ((37, 5, 64), 6, (2,)) in graphs and ((9, 9, 9), 0, (1,)) in graphs, list(graphs)
    lm.model.check_device_errors()
    cache.book.audit()


def test_layouts_that_take_turns_do_not_evict_each_other_for_ever(cuda, model_folders):
    """Three layouts of which only one fits the rows kept as captured steps, coming by in turn: the first to
    come back is captured and stays, the others run eagerly every time (a capture costs far more than a replay
    saves, so capturing and dropping them in turn would be the worst of both). A fourth layout that then comes
    by more often than the kept one takes its place. Every step's logits are checked."""
    import camelid_b200
    from camelid_b200 import StepEntry
    from camelid_b200.engine import graphs as graphs_mod
    from camelid_b200.options import KernelOptions
    name, dtype = "tiny_b", "float32"
    lm = camelid_b200.load(model_folders[name], dtype=dtype, options=KernelOptions(captured_step_rows=128))
    vocab = CONFIGS[name]["vocab_size"]
    cache = lm.new_cache(256, max_slots=2)
    captured = []
    real = graphs_mod.StepGraph.run_and_capture

    def counting(self):
        captured.append(self.rows)
        return real(self)

    graphs_mod.StepGraph.run_and_capture = counting
    try:
        def run(n, seed):
            ids = tokens(seed, n, vocab)
            slot = cache.alloc_slot()
            got = lm.step(cache, [StepEntry(slot, ids, [n - 1])]).cpu()
            cache.free_slot(slot)
            assert_close(got, oracle(model_folders[name], ids)[n - 1:], dtype, f"{n} tokens, seed {seed}")

        for turn in range(5):
            for n in (100, 90, 80):
                run(n, 300 + 10 * turn + n)
        assert captured == [100], captured
        for again in range(8):
            run(70, 500 + again)
        assert captured == [100, 70], captured
        kept = lm.model._step_graphs[cache]
        assert [k[0] for k in kept] == [(70,)], list(kept)
    finally:
        graphs_mod.StepGraph.run_and_capture = real
    lm.model.check_device_errors()
    cache.book.audit()


def test_sampled_generation_fed_on_the_device(cuda, model_folders):
    """Temperature sampling (with top-k and top-p) also decodes with the token fed back on the
    device: the draw of each step is made there from the seed and the row's position, the same
    number the host makes, so the tokens are those of the loop that reads every token back, for three
    seeds and settings through one captured graph per batch shape, and a request's tokens do not depend on its batch."""
    import camelid_b200
    from camelid_b200 import KernelOptions
    name = "tiny_a"
    prompts = [tokens(50 + i, n, CONFIGS[name]["vocab_size"]) for i, n in enumerate([5, 11, 1, 30])]
    fed = camelid_b200.load(model_folders[name], dtype="float32")
    unfed = camelid_b200.load(model_folders[name], dtype="float32", options=KernelOptions(feed_on_device=False))
    runs = []
    real = fed.model.decode_fed
    fed.model.decode_fed = lambda *a, **k: (runs.append(a[3]), real(*a, **k))[1]
    for kw in (dict(temperature=0.8, seed=1234), dict(temperature=1.3, top_k=40, top_p=0.9, seed=2 ** 63 + 11),
               dict(temperature=0.7, min_p=0.05, seed=0)):
        a = fed.generate(prompts, max_tokens=30, stop_token_ids=(), **kw)
        b = unfed.generate(prompts, max_tokens=30, stop_token_ids=(), **kw)
        assert a == b, kw
        assert fed.generate(prompts[::-1], max_tokens=30, stop_token_ids=(), **kw) == a[::-1]
    assert runs and all(r == 29 for r in runs)
    # temperature and the filters reach the kernel through device memory: the three settings shared their graphs
    sampled = [k for g in fed.model._graphs.values() for k in g if k[2] == "sample"]
    assert sampled and len(sampled) == len({k[:2] for k in sampled}), sampled
    cfg, w = pl.read_model(model_folders[name])
    want = pl.generate(cfg, w, prompts[:2], 12, temperature=0.8, seed=1234, dtype=torch.float64)
    assert fed.generate(prompts[:2], max_tokens=12, temperature=0.8, seed=1234, stop_token_ids=()) == want
