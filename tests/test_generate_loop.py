"""The generation loop's decisions, with stand-ins for model, cache and sampler: batches
that fit, stop tokens (kept), sequences that end earlier, budgets, slots given back."""
import pytest

from camelid_b200 import CacheError, StepError
from camelid_b200.cache import CacheBook, KVSpec
from camelid_b200.engine.generate import generate, plan_batches, token_budget


class FakeCache:
    def __init__(self, n_pages, n_slots, max_position=10_000):
        self.book = CacheBook([KVSpec(1, 16)], n_pages, n_slots, max_position)
        self.max_live = 0

    def alloc_slot(self):
        s = self.book.alloc_slot()
        self.max_live = max(self.max_live, self.book.slots.n_held)
        return s

    def free_slot(self, s):
        self.book.free_slot(s)


class FakeModel:
    """Next token = (last token + 1) % 100; remembers every step it was asked to run."""

    def __init__(self):
        self.steps = []

    def step(self, cache, entries):
        cache.book.check_extend([(e.slot, len(e.tokens)) for e in entries])
        for e in entries:
            cache.book.extend(e.slot, len(e.tokens))
            cache.book.commit(e.slot, len(e.tokens))
            assert e.want == [len(e.tokens) - 1]
        self.steps.append([(e.slot, list(e.tokens)) for e in entries])
        return [(e.tokens[-1] + 1) % 100 for e in entries]


class FakeSampler:
    def __init__(self):
        self.histories = []

    def sample(self, logits, histories):
        self.histories.append([list(h) for h in histories])
        return list(logits)


def test_token_budget_and_batches():
    assert token_budget(10, 5, 100, 4) == 5
    assert token_budget(98, 5, 100, 4) == 3            # positions 98, 99 fed; the last token is not
    assert token_budget(100, 5, 100, 4) == 1
    assert token_budget(250, 50, 1000, 4) == 7         # a cache of 256 tokens
    assert plan_batches([10, 10, 10], [5, 5, 5], 8, 8, None) == [[0, 1, 2]]
    assert plan_batches([10, 10, 10], [5, 5, 5], 8, 8, 2) == [[0, 1], [2]]
    assert plan_batches([100, 100, 10], [29, 29, 5], 4, 8, None) == [[0, 1], [2]]
    assert plan_batches([100, 100, 10], [29, 30, 5], 4, 8, None) == [[0], [1, 2]]
    assert plan_batches([10, 10, 10], [5, 5, 5], 8, 2, None) == [[0, 1], [2]]
    with pytest.raises(CacheError):
        plan_batches([300], [1], 4, 4, None)


def test_unequal_prompts_stop_and_length():
    model, cache, sampler = FakeModel(), FakeCache(16, 8), FakeSampler()
    out = generate(model, cache, sampler, [[1, 2, 3], [50], [7, 8]], 5, stop_ids={53, 10})
    assert out[0].tokens == [4, 5, 6, 7, 8] and out[0].finish_reason == "length"
    assert out[1].tokens == [51, 52, 53] and out[1].finish_reason == "stop"        # the stop token is kept
    assert out[2].tokens == [9, 10] and out[2].finish_reason == "stop"
    assert [o.prompt_tokens for o in out] == [3, 1, 2]
    # one step for all prompts, then one token per live sequence; ended ones leave at once
    assert [len(s) for s in model.steps] == [3, 3, 2, 1, 1]
    assert model.steps[0] == [(0, [1, 2, 3]), (1, [50]), (2, [7, 8])]
    assert model.steps[2] == [(0, [5]), (1, [52])]
    # the sampler sees prompt plus generated tokens of each live sequence
    assert sampler.histories[1] == [[1, 2, 3, 4], [50, 51], [7, 8, 9]]
    assert cache.book.slots.n_held == 0 and cache.book.pools[0].n_held == 0
    cache.book.audit()


def test_batches_one_after_another_reuse_slots():
    model, cache, sampler = FakeModel(), FakeCache(4, 2), FakeSampler()
    prompts = [[i] for i in range(5)]
    out = generate(model, cache, sampler, prompts, [1, 2, 3, 1, 2])
    assert [o.tokens for o in out] == [[1], [2, 3], [3, 4, 5], [4], [5, 6]]
    assert cache.max_live == 2
    slots_used = [slot for step in model.steps for slot, _ in step]
    assert set(slots_used) == {0, 1}
    assert cache.book.slots.n_held == 0
    assert model.steps[0] == [(0, [0]), (1, [1])] and model.steps[1] == [(1, [2])]
    assert model.steps[2] == [(0, [2]), (1, [3])]            # the next batch starts in the same slots


def test_capacity_ends_a_sequence():
    model, cache, sampler = FakeModel(), FakeCache(1, 1, max_position=70), FakeSampler()
    out = generate(model, cache, sampler, [list(range(60))], 50)
    assert out[0].finish_reason == "capacity" and len(out[0].tokens) == 5     # 64 cached positions
    out = generate(model, cache, sampler, [list(range(60))], 3)
    assert out[0].finish_reason == "length" and len(out[0].tokens) == 3
    out = generate(model, cache, sampler, [[1]], 0)
    assert out[0].tokens == [] and out[0].finish_reason == "length"


def test_bad_requests_and_failures_leave_no_slot_behind():
    model, cache, sampler = FakeModel(), FakeCache(4, 4, max_position=100), FakeSampler()
    with pytest.raises(StepError):
        generate(model, cache, sampler, [[]], 4)
    with pytest.raises(StepError):
        generate(model, cache, sampler, [[1]], [1, 2])
    with pytest.raises(StepError):
        generate(model, cache, sampler, [list(range(101))], 4)
    assert generate(model, cache, sampler, [], 4) == []

    class Boom(FakeModel):
        def step(self, cache, entries):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step(cache, entries)
    with pytest.raises(RuntimeError):
        generate(Boom(), cache, sampler, [[1], [2]], 10)
    assert cache.book.slots.n_held == 0 and cache.book.pools[0].n_held == 0


class FedModel(FakeModel):
    """A stand-in that decodes runs of steps on its own, as a model with captured graphs does:
    every run is remembered as (slots, first tokens, steps)."""
    use_graphs = True

    class options:
        feed_on_device = True

    def __init__(self):
        super().__init__()
        self.runs = []

    def decode_natively(self, *a, **k):
        raise AssertionError("a batch without penalties must take the fed loop")

    def decode_fed(self, cache, slots, tokens, steps, sampling=None):
        import numpy as np
        cache.book.check_extend([(s, steps) for s in slots])
        for s in slots:
            cache.book.extend(s, steps)
            cache.book.commit(s, steps)
        self.runs.append((list(slots), list(tokens), steps))
        return np.array([[(t + 1 + k) % 100 for t in tokens] for k in range(steps)], dtype=np.int32)


class GreedySampler(FakeSampler):
    native_ok = True
    error_word = None

    class options:
        greedy = True


def test_greedy_batches_run_on_the_device_and_cut_at_stop_tokens():
    from camelid_b200.engine.generate import FED_RUN_WITH_STOPS
    model, cache, sampler = FedModel(), FakeCache(64, 8), GreedySampler()
    # without stop tokens: one run for everything the shortest budget allows, then the rest
    out = generate(model, cache, sampler, [[1, 2, 3], [50]], [40, 6])
    assert out[0].tokens == [(4 + k) % 100 for k in range(40)] and out[0].finish_reason == "length"
    assert out[1].tokens == [51, 52, 53, 54, 55, 56] and out[1].finish_reason == "length"
    assert model.runs == [([0, 1], [4, 51], 5), ([0], [9], 34)]
    assert cache.book.slots.n_held == 0 and cache.book.pools[0].n_held == 0
    # with stop tokens: short runs; what a sequence produced after its stop token is dropped
    model = FedModel()
    out = generate(model, cache, sampler, [[1, 2, 3], [50]], 60, stop_ids={57})
    assert out[1].tokens == [51, 52, 53, 54, 55, 56, 57] and out[1].finish_reason == "stop"
    assert out[0].tokens == [(4 + k) % 100 for k in range(54)] and out[0].tokens[-1] == 57 and out[0].finish_reason == "stop"
    assert [r[2] for r in model.runs] == [FED_RUN_WITH_STOPS] * 3 + [60 - 1 - 3 * FED_RUN_WITH_STOPS]
    assert model.runs[1][0] == [0]                       # the stopped sequence left after the first run
    cache.book.audit()
    assert cache.book.slots.n_held == 0 and cache.book.pools[0].n_held == 0
