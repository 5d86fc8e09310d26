"""Typed configuration of the dense Llama decoder, read from config.json's own keys.

The reference's typed configuration is ``LlamaModelConfig`` (src/model.rs:9-52) with its
Hugging Face twin (src/model_source.rs:49-68, keys probed at :345-361). The defaults and
the checks follow it: kv heads default to the heads (src/model.rs:698-705), head_dim to
hidden/heads (src/model.rs:1405-1456), theta to 10000 (src/inference/rope.rs:174-180),
llama3 scaling to low 1 / high 4 / original 8192 (src/inference/rope.rs:413-422); the
geometry checks are those of src/model.rs:1409-1437 and the scaling checks those of
src/inference/rope.rs:377-459. Unlike the reference's stub (src/model_source.rs:551-557)
``rope_scaling`` of type ``llama3`` is accepted.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict
from typing import Any, Optional

from ..errors import ConfigError

_MISSING = object()


def _get(d: dict, key: str, typ, default=_MISSING, *, positive=False, finite=True):
    """One key of config.json, with its type and range checked and the key named in the error."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(key, "required key is missing")
        return default
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise ConfigError(key, f"expected an integer, got {v!r}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(key, f"expected a number, got {v!r}")
        v = float(v)
        if finite and not math.isfinite(v):
            raise ConfigError(key, f"expected a finite number, got {v!r}")
    elif typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(key, f"expected true or false, got {v!r}")
    elif typ is str:
        if not isinstance(v, str):
            raise ConfigError(key, f"expected a string, got {v!r}")
    if positive and not v > 0:
        raise ConfigError(key, f"must be greater than zero, got {v!r}")
    return v


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json. ``rope_type`` is "llama3" (the only law this
    architecture uses) with its four constants."""
    rope_type: str
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @classmethod
    def from_dict(cls, d: Any) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise ConfigError("rope_scaling", f"expected an object, got {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError("rope_scaling.rope_type", f"{kind!r} is not supported (known: 'llama3', 'default')")
        sub = {f"rope_scaling.{k}": v for k, v in d.items()}
        factor = _get(sub, "rope_scaling.factor", float, positive=True)
        low = _get(sub, "rope_scaling.low_freq_factor", float, 1.0, positive=True)
        high = _get(sub, "rope_scaling.high_freq_factor", float, 4.0, positive=True)
        orig = _get(sub, "rope_scaling.original_max_position_embeddings", int, 8192, positive=True)
        if not high > low:
            raise ConfigError("rope_scaling.high_freq_factor", f"must be greater than low_freq_factor ({low}), got {high}")
        return cls("llama3", factor, low, high, orig)

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of the model; nothing of this stands in code elsewhere."""
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Any = None            # an integer, a list of integers, or None
    architecture: str = "LlamaForCausalLM"
    extra: dict = field(default_factory=dict, compare=False)

    # ---- derived sizes (src/model.rs:1391-1457) ----
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def stop_token_ids(self) -> tuple:
        e = self.eos_token_id
        if e is None:
            return ()
        return tuple(e) if isinstance(e, (list, tuple)) else (int(e),)

    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        if not isinstance(d, dict):
            raise ConfigError("<root>", "config.json must hold an object")
        model_type = d.get("model_type")
        if model_type is not None and model_type != "llama":
            raise ConfigError("model_type", f"expected 'llama', got {model_type!r}")
        hidden = _get(d, "hidden_size", int, positive=True)
        heads = _get(d, "num_attention_heads", int, positive=True)
        kv_heads = _get(d, "num_key_value_heads", int, heads, positive=True)
        head_dim = _get(d, "head_dim", int, None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError("hidden_size", f"{hidden} is not a multiple of num_attention_heads ({heads}) and head_dim is not given")
            head_dim = hidden // heads
        if head_dim <= 0:
            raise ConfigError("head_dim", f"must be greater than zero, got {head_dim}")
        if head_dim % 2 != 0:
            raise ConfigError("head_dim", f"rotary pairs need an even head_dim, got {head_dim}")
        if heads % kv_heads != 0:
            raise ConfigError("num_key_value_heads", f"{kv_heads} does not divide num_attention_heads ({heads})")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError("hidden_act", f"this architecture's feed-forward is SwiGLU ('silu'), got {act!r}")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(key, "biases are not part of this architecture")
        if d.get("sliding_window") is not None:
            raise ConfigError("sliding_window", "this architecture attends to all keys")
        theta = _get(d, "rope_theta", float, 10000.0, positive=True)
        eps = _get(d, "rms_norm_eps", float, positive=True)
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            raise ConfigError("torch_dtype", f"expected 'bfloat16', 'float16' or 'float32', got {dtype!r}")
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        known = {f.name for f in cls.__dataclass_fields__.values()} | {
            "model_type", "architectures", "hidden_act", "attention_bias", "mlp_bias", "sliding_window", "dtype"}
        return cls(
            vocab_size=_get(d, "vocab_size", int, positive=True),
            hidden_size=hidden,
            num_hidden_layers=_get(d, "num_hidden_layers", int, positive=True),
            intermediate_size=_get(d, "intermediate_size", int, positive=True),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_get(d, "max_position_embeddings", int, positive=True),
            rms_norm_eps=eps,
            rope_theta=theta,
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            torch_dtype=dtype,
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id"),
            architecture=archs[0],
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict:
        """The config.json that ``from_dict`` reads back to an equal configuration."""
        out = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out
