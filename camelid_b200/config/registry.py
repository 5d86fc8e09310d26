"""One registry from the architecture's name in config.json to its model.

The reference gates on ``general.architecture`` by a string match
(src/model.rs:60-74, :78-132) and, for Hugging Face folders, on
``architectures`` holding "LlamaForCausalLM" (src/model_source.rs:529-541); an unknown
name is a typed error that lists the known ones.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable

from ..errors import ConfigError, UnknownArchitectureError
from .llama import LlamaConfig
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable      # dict -> typed configuration
    make_plan: Callable         # typed configuration -> ModelPlan


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable, make_plan: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, parse_config, make_plan)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(config_dict: dict) -> Architecture:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("architectures", "required key is missing (a list with the model class name)")
    for name in archs:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise UnknownArchitectureError(
        f"no model is registered for architectures {archs!r}; known: {known_architectures()}")


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError("<file>", f"{path} does not exist")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError("<file>", f"{path} is not valid JSON: {e}") from None


def load_config(folder_or_dict):
    """(architecture, typed configuration, plan) of a model folder or a config dict."""
    d = read_config_json(folder_or_dict) if isinstance(folder_or_dict, (str, os.PathLike)) else folder_or_dict
    arch = architecture_of(d)
    cfg = arch.parse_config(d)
    return arch, cfg, arch.make_plan(cfg)


# ---------------------------------------------------------------------------------------
# the one architecture of this library


def llama_plan(cfg: LlamaConfig) -> ModelPlan:
    """The dense Llama decoder as parts: RMSNorm, grouped-query attention with rotary
    positions (split-half pairs for un-permuted weights, src/inference/rope.rs:501-509),
    RMSNorm, SwiGLU; every layer once, in order; final norm; output projection that is the
    embedding when tied (src/model.rs:772-775)."""
    rope = PartSpec("rope", {
        "rotary_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
    })
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
        layers.append(LayerSpec(
            arrangement="prenorm",
            norm1=PartSpec("rmsnorm", norm, p + "input_layernorm."),
            mixer=PartSpec("attention", {
                "hidden_size": cfg.hidden_size,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "position": rope,
                "window": None,
            }, p + "self_attn."),
            norm2=PartSpec("rmsnorm", norm, p + "post_attention_layernorm."),
            ffn=PartSpec("swiglu", {
                "hidden_size": cfg.hidden_size,
                "intermediate_size": cfg.intermediate_size,
            }, p + "mlp."),
        ))
    return ModelPlan(
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                           "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm."),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                  "tied_to": "model.embed_tokens." if cfg.tie_word_embeddings else None},
                      "lm_head."),
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        stop_token_ids=cfg.stop_token_ids,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_plan)
