"""Writes tests/golden/plain_micro.json: logits of the plain implementation
(tests/plain_llama.py) for a micro model whose weights come from a linear congruential
generator written out here, so that they do not depend on any library's random numbers.

The plain implementation rests on the reference's formulas (its Rust code cannot be
compiled here: no Rust toolchain), so this file pins the oracle against itself: a change
of the oracle that moves these numbers has to be deliberate. Run from the repository root:

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import plain_llama as pl  # noqa: E402

CONFIG = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 24, "hidden_size": 16,
          "num_hidden_layers": 2, "intermediate_size": 40, "num_attention_heads": 4, "num_key_value_heads": 2,
          "head_dim": 4, "max_position_embeddings": 64, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
          "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                           "original_max_position_embeddings": 16}, "tie_word_embeddings": False}
TOKENS = [3, 17, 0, 23, 8, 8, 5, 12, 1, 19]


def lcg_weights(cfg):
    """Uniform values in [-0.25, 0.25) from x <- (1103515245 x + 12345) mod 2^31, in name order;
    norm weights are 1 plus such a value."""
    state = [20261125]

    def draw(n):
        out = np.empty(n, dtype=np.float64)
        x = state[0]
        for i in range(n):
            x = (1103515245 * x + 12345) % (1 << 31)
            out[i] = x / float(1 << 31) * 0.5 - 0.25
        state[0] = x
        return out

    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,), "lm_head.weight": (v, h)}
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes.update({p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
                       p + "self_attn.q_proj.weight": (q, h), p + "self_attn.k_proj.weight": (kv, h),
                       p + "self_attn.v_proj.weight": (kv, h), p + "self_attn.o_proj.weight": (h, q),
                       p + "mlp.gate_proj.weight": (i, h), p + "mlp.up_proj.weight": (i, h),
                       p + "mlp.down_proj.weight": (h, i)})
    w = {}
    for name in sorted(shapes):
        vals = draw(int(np.prod(shapes[name])))
        if name.endswith("norm.weight"):
            vals = vals + 1.0
        w[name] = torch.tensor(vals.reshape(shapes[name]), dtype=torch.float64)
    return w


def compute():
    w = lcg_weights(CONFIG)
    logits = pl.forward(CONFIG, w, TOKENS, dtype=torch.float64)
    return {"config": CONFIG, "tokens": TOKENS, "logits_last": [round(float(x), 10) for x in logits[-1]],
            "logits_first": [round(float(x), 10) for x in logits[0]],
            "argmax_per_position": [int(x) for x in logits.argmax(dim=-1)],
            "sum_abs": round(float(logits.abs().sum()), 8)}


if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_micro.json")
    with open(out, "w") as f:
        json.dump(compute(), f, indent=1)
    print("wrote", out)
