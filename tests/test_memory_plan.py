"""The memory plan: bytes of weights, cache and workspace from a configuration alone, and the
refusal before anything is allocated."""
import pytest
import torch

import camelid_b200
from camelid_b200 import MemoryBudgetError, benchmark, memory_plan
from conftest import TINY_A, TINY_B


def test_plan_counts_what_the_survey_counts():
    """Llama 3.2 1B: 973.1 M linear + 262.7 M embedding (tied) + 67.6 k norm parameters; the
    cache keeps 2 * 16 layers * 8 kv heads * 64 = 16,384 elements a position."""
    cfg = benchmark.config_for(2)
    p = memory_plan(cfg, "bfloat16", max_tokens=8 * 4096, max_slots=8)
    assert p.weights == (973_078_528 + 262_668_288 + 33 * 2048) * 2
    assert p.cache == 8 * 4096 * 16_384 * 2
    assert p.total == p.weights + p.cache + p.workspace and 0 < p.workspace < 1 << 30
    f = memory_plan(cfg, "float32", max_tokens=8 * 4096, max_slots=8)
    assert f.weights == 2 * p.weights and f.cache == 2 * p.cache
    untied = memory_plan({**cfg, "tie_word_embeddings": False}, "bfloat16")
    assert untied.weights - p.weights == 262_668_288 * 2 and untied.cache == 0
    # tokens are rounded up to pages of 64
    assert memory_plan(TINY_A, "float32", max_tokens=65).cache == memory_plan(TINY_A, "float32", max_tokens=128).cache


def test_8b_in_float32_is_refused_on_a_32_gb_device_with_the_numbers():
    cfg = benchmark.config_for(4)
    plan = memory_plan(cfg, "float32", max_tokens=8 * 8192, max_slots=8)
    assert 32.0e9 < plan.weights < 32.3e9                      # 8.03 G parameters in 4 bytes
    with pytest.raises(MemoryBudgetError) as e:
        plan.check(32 * 2 ** 30, "Llama 3.1 8B in float32")
    assert e.value.needed == plan.total and e.value.available == 32 * 2 ** 30
    assert f"{plan.weights:,}" in str(e.value) and f"{plan.cache:,}" in str(e.value)
    plan.check(64 * 2 ** 30)
    assert isinstance(e.value, camelid_b200.CacheError) and isinstance(e.value, camelid_b200.CamelidError)


def test_load_refuses_before_it_reads_a_tensor():
    """``load_tensors`` checks names, shapes and then the bytes: a source whose tensors would
    not fit is refused without one tensor having been asked for."""
    from camelid_b200 import DecoderModel
    model = DecoderModel.from_config(TINY_B, dtype=torch.float32, device="cpu")
    specs = model.tensor_specs()

    class Source:
        asked = []

        def names(self):
            return list(specs)

        def shape(self, name):
            return list(specs[name].shape)

        def dtype(self, name):
            return torch.bfloat16

        def tensor(self, name):
            self.asked.append(name)
            raise AssertionError("no tensor may be read")
    src = Source()
    need = model.memory_plan().weights
    with pytest.raises(MemoryBudgetError) as e:
        model.load_tensors(src, available_bytes=need - 1)
    assert src.asked == [] and not model.loaded and e.value.needed == need
