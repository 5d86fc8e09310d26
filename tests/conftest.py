"""Shared fixtures: the two tiny configurations of the architecture that differ in every size
and option (tiny_a and tiny_b), and three more with sizes that are harder for the kernels,
written as model folders with random weights into a temporary folder."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 2, "intermediate_size": 160,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "max_position_embeddings": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": True,
    "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 512, "hidden_size": 192, "num_hidden_layers": 3, "intermediate_size": 512,
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32, "max_position_embeddings": 256,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "tie_word_embeddings": False, "eos_token_id": [3, 11],
}
# the same with a vocabulary and a feed-forward width that are no multiple of 8: nothing fills a tile
TINY_B_ODD = {**TINY_B, "vocab_size": 517, "intermediate_size": 520}
# a third shape for long decoding and the first tokens of a sequence: more heads than a
# block's warps per kv head, a head size that is no power of two, a long context
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 300, "hidden_size": 96, "num_hidden_layers": 2, "intermediate_size": 136,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "max_position_embeddings": 1024,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "tie_word_embeddings": True,
}
# a fourth with the head size of the tensor-core attention kernels (64), three query heads to
# a kv head, and a width, feed-forward and vocabulary that fill no tile
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 331, "hidden_size": 200, "num_hidden_layers": 2, "intermediate_size": 328,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "max_position_embeddings": 2048,
    "rms_norm_eps": 2e-5, "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "tie_word_embeddings": False, "eos_token_id": 2,
}
CONFIGS = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_b_odd": TINY_B_ODD, "tiny_c": TINY_C, "tiny_d": TINY_D}
SEEDS = {"tiny_a": 0, "tiny_b": 1, "tiny_b_odd": 1, "tiny_c": 5, "tiny_d": 9}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (bfloat16 weights; tiny_b keeps
    its norm weights in float32)."""
    import torch
    from camelid_b200.weights.random_init import write_random_model
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(tmp_path_factory.mktemp(name))
        write_random_model(d, cfg, SEEDS[name], torch.bfloat16,
                           norm_dtype=torch.float32 if name.startswith("tiny_b") else None)
        out[name] = d
    return out


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
