"""Configuration and registry: keys, defaults, ranges, and the error for each."""
import copy
import json

import pytest

from camelid_b200 import ConfigError, LlamaConfig, UnknownArchitectureError, load_config
from camelid_b200.config import known_architectures, register_architecture
from conftest import TINY_A, TINY_B


def test_parse_tiny_configs_and_round_trip():
    for d in (TINY_A, TINY_B):
        cfg = LlamaConfig.from_dict(d)
        assert cfg.vocab_size == d["vocab_size"] and cfg.head_dim == d["head_dim"]
        assert cfg.q_width == d["num_attention_heads"] * d["head_dim"]
        assert cfg.kv_width == d["num_key_value_heads"] * d["head_dim"]
        assert LlamaConfig.from_dict(cfg.to_dict()) == cfg
    b = LlamaConfig.from_dict(TINY_B)
    assert b.rope_scaling.rope_type == "llama3" and b.rope_scaling.original_max_position_embeddings == 64
    assert b.stop_token_ids == (3, 11) and LlamaConfig.from_dict(TINY_A).stop_token_ids == (7,)


def test_defaults():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta",
                                                        "tie_word_embeddings", "rope_scaling")}
    cfg = LlamaConfig.from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads          # src/model.rs:698-705
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads  # src/model.rs:1405-1456
    assert cfg.rope_theta == 10000.0 and cfg.tie_word_embeddings is False and cfg.rope_scaling is None
    s = LlamaConfig.from_dict({**TINY_A, "rope_scaling": {"rope_type": "llama3", "factor": 8}}).rope_scaling
    assert (s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == (1.0, 4.0, 8192)


@pytest.mark.parametrize("key,value", [
    ("vocab_size", 0), ("hidden_size", -1), ("num_hidden_layers", 0), ("intermediate_size", "x"),
    ("num_attention_heads", 0), ("num_key_value_heads", 3), ("head_dim", 15), ("rms_norm_eps", 0.0),
    ("rms_norm_eps", float("nan")), ("rope_theta", -1.0), ("max_position_embeddings", 0), ("hidden_act", "gelu"),
    ("attention_bias", True), ("mlp_bias", True), ("sliding_window", 128), ("tie_word_embeddings", "yes"),
    ("torch_dtype", "int8"), ("model_type", "mistral"),
    ("rope_scaling", {"rope_type": "yarn", "factor": 2.0}), ("rope_scaling", {"rope_type": "llama3"}),
    ("rope_scaling", {"rope_type": "llama3", "factor": 0.0}),
    ("rope_scaling", {"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 4.0, "high_freq_factor": 4.0}),
])
def test_bad_values_name_their_key(key, value):
    d = copy.deepcopy(TINY_A)
    d[key] = value
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert key.split(".")[0] in str(e.value)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "intermediate_size",
                                 "num_attention_heads", "max_position_embeddings", "rms_norm_eps"])
def test_missing_required_key(key):
    d = {k: v for k, v in TINY_A.items() if k != key}
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert e.value.key == key


def test_hidden_not_multiple_of_heads_needs_head_dim():
    d = {**TINY_A, "hidden_size": 66}
    LlamaConfig.from_dict(d)                        # head_dim given: fine
    d.pop("head_dim")
    with pytest.raises(ConfigError):
        LlamaConfig.from_dict(d)


def test_registry(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    arch, cfg, plan = load_config(TINY_B)
    assert arch.name == "LlamaForCausalLM" and len(plan.layers) == 3 and len(plan.schedule) == 3
    assert plan.layers[1].mixer.params["num_kv_heads"] == 1 and plan.layers[1].ffn.params["intermediate_size"] == 512
    assert plan.head.params["tied_to"] is None
    assert load_config(TINY_A)[2].head.params["tied_to"] == "model.embed_tokens."
    with pytest.raises(UnknownArchitectureError) as e:
        load_config({**TINY_A, "architectures": ["GPT2LMHeadModel"]})
    assert "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        load_config({k: v for k, v in TINY_A.items() if k != "architectures"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert load_config(str(tmp_path))[1].vocab_size == 256
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nowhere"))


def test_another_architecture_registers_without_touching_the_library():
    from camelid_b200.config import llama_plan
    register_architecture("ToyForCausalLM", LlamaConfig.from_dict, llama_plan)
    arch, _cfg, _plan = load_config({**TINY_A, "architectures": ["ToyForCausalLM"]})
    assert arch.name == "ToyForCausalLM"


def test_plan_rejects_bad_schedule():
    from camelid_b200.config import ModelPlan, ScheduleEntry
    _a, _c, plan = load_config(TINY_A)
    kw = {f: getattr(plan, f) for f in plan.__dataclass_fields__}
    for bad in ([ScheduleEntry(5)], [ScheduleEntry(0, 0)], [ScheduleEntry(0), ScheduleEntry(1, 0), ScheduleEntry(1, 1)]):
        with pytest.raises(ConfigError):
            ModelPlan(**{**kw, "schedule": tuple(bad)})
    ModelPlan(**{**kw, "schedule": (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, 1))})
