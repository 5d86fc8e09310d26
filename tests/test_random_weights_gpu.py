"""Random weights drawn on the device are the numbers the host computes, bit for bit."""
import pytest
import torch

from conftest import CONFIGS, SEEDS
from helpers import tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_every_tensor_host_equals_device(cuda, name, dtype):
    from camelid_b200 import DecoderModel
    from camelid_b200.weights.random_init import random_tensors
    specs = DecoderModel.from_config(CONFIGS[name], dtype=dtype, device="cpu").tensor_specs()
    host = random_tensors(specs, SEEDS[name], dtype, "cpu")
    dev = random_tensors(specs, SEEDS[name], dtype, cuda)
    assert set(host) == set(dev)
    for n in specs:
        assert dev[n].dtype == dtype and dev[n].shape == host[n].shape
        assert torch.equal(dev[n].cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                           host[n].view(torch.int16 if dtype == torch.bfloat16 else torch.int32)), n


def test_a_slice_of_the_benchmark_embedding(cuda):
    """A million elements in the middle of the embedding of the Llama 3.2 1B shape under the
    benchmark's seed: the device's fill of the whole tensor against the host's slice."""
    from camelid_b200.parts.base import TensorSpec
    from camelid_b200.weights.random_init import random_slice, random_tensor
    name, seed, first, count = "model.embed_tokens.weight", 2, 128256 * 2048 // 2 - 12345, 1 << 20
    dev = random_tensor(name, TensorSpec((128256, 2048), "embedding"), seed, torch.float32, cuda)
    host = random_slice(name, "embedding", seed, first, count)
    assert torch.equal(dev.view(-1)[first:first + count].cpu().view(torch.int32), host.view(torch.int32))
    tail = random_slice(name, "embedding", seed, 128256 * 2048 - 1000, 1000)
    assert torch.equal(dev.view(-1)[-1000:].cpu(), tail)
    assert abs(float(dev.std()) - 0.02) < 1e-4 and abs(float(dev.mean())) < 1e-5


def test_from_random_is_the_folder_written_on_the_host(cuda, tmp_path):
    """``from_random`` (drawn on the device) and ``load`` of the folder ``write_random_model``
    writes on the CPU are the same model: equal logits to the bit."""
    import camelid_b200
    from camelid_b200 import StepEntry
    cfg = CONFIGS["tiny_b"]
    folder = camelid_b200.write_random_model(str(tmp_path / "m"), cfg, 21, torch.float32)
    ids = tokens(3, 50, cfg["vocab_size"])
    out = []
    for lm in (camelid_b200.load(folder, dtype="float32"), camelid_b200.from_random(cfg, 21, dtype="float32")):
        cache = lm.new_cache(64)
        out.append(lm.step(cache, [StepEntry(cache.alloc_slot(), ids, list(range(50)))]).cpu())
    assert torch.equal(out[0], out[1])
