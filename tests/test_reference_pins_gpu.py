"""The engine's cache against the numbers the reference's own session test expects
(tests/inference_session.rs:27-56), on that test's model widened to a head size the kernels
take: hidden 32, two heads on one kv head of 16, matrices that select columns. Token 1 is
0.5 in column 0, token 2 is 1 in column 8, which the split-half rotation pairs with column 0
at frequency 1, so the kept key of token 2 at position 1 is (-y sin 1, ..., y cos 1) as there.
Column 31, which no key or value reads, carries what brings each token's mean square to the
reference's (0.0625 and 0.25), so the expected numbers are the reference's own digits."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _select_rows(rows, cols, source_cols, scale=1.0):
    m = torch.zeros(rows, cols)
    for r, c in enumerate(source_cols):
        m[r, c] = scale
    return m


def _model(dtype):
    from camelid_b200 import DecoderModel, LanguageModel
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 3, "hidden_size": 32,
           "num_hidden_layers": 1, "intermediate_size": 48, "num_attention_heads": 2, "num_key_value_heads": 1,
           "head_dim": 16, "max_position_embeddings": 64, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
           "tie_word_embeddings": False}
    emb = torch.zeros(3, 32)
    emb[0, 0], emb[1, 0], emb[2, 8] = 1.0, 0.5, 1.0
    emb[1, 31], emb[2, 31] = math.sqrt(0.0625 * 32 - 0.25), math.sqrt(0.25 * 32 - 1.0)
    p = "model.layers.0."
    w = {"model.embed_tokens.weight": emb, "model.norm.weight": torch.ones(32), "lm_head.weight": _select_rows(3, 32, [0, 1, 2]),
         p + "input_layernorm.weight": torch.ones(32), p + "post_attention_layernorm.weight": torch.ones(32),
         p + "self_attn.q_proj.weight": _select_rows(32, 32, list(range(32))),
         p + "self_attn.k_proj.weight": _select_rows(16, 32, list(range(16))),
         p + "self_attn.v_proj.weight": _select_rows(16, 32, list(range(16)), 0.5),
         p + "self_attn.o_proj.weight": _select_rows(32, 32, list(range(32))),
         p + "mlp.gate_proj.weight": _select_rows(48, 32, list(range(32)) + list(range(16))),
         p + "mlp.up_proj.weight": _select_rows(48, 32, list(range(32)) + list(range(16))),
         p + "mlp.down_proj.weight": _select_rows(32, 48, list(range(32)))}
    model = DecoderModel.from_config(cfg, dtype=dtype, device="cuda")
    model.load_tensors(w)
    return LanguageModel(model)


@pytest.mark.parametrize("cut", ["token by token", "one prompt"])
def test_kept_keys_and_values_are_the_reference_sessions(cuda, cut):
    from camelid_b200 import StepEntry
    lm = _model("float32")
    cache = lm.new_cache(64, max_slots=1)
    slot = cache.alloc_slot()
    if cut == "one prompt":
        lm.step(cache, [StepEntry(slot, [1, 2], [1])])
    else:
        lm.step(cache, [StepEntry(slot, [1], [0])])
        lm.step(cache, [StepEntry(slot, [2], [0])])
    page = cache.book.pages[0][slot][0]
    _group, k_pages, v_pages = cache.kv_pages(0)
    k, v = k_pages[page, 0].float().cpu(), v_pages[page, 0].float().cpu()      # [64 positions, 16]
    y = 1.0 / math.sqrt(0.25 + 1e-6)
    assert abs(float(k[0, 0]) - 1.999984) < 5e-4 and float(k[0, 1:].abs().max()) < 5e-4
    assert abs(float(v[0, 0]) - 0.999992) < 5e-4 and float(v[0, 1:].abs().max()) < 5e-4
    assert abs(float(k[1, 0]) + y * math.sin(1.0)) < 5e-4
    assert abs(float(k[1, 8]) - y * math.cos(1.0)) < 5e-4
    rest = k[1].clone()
    rest[0] = rest[8] = 0
    assert float(rest.abs().max()) < 5e-4
    assert abs(float(v[1, 8]) - 0.5 * y) < 5e-4
    cache.free_slot(slot)
