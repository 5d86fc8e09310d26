"""The Python entry point: load a model folder, generate, or drive the step function.

    import camelid_b200
    lm = camelid_b200.load("model_dir", dtype="bfloat16")
    out = lm.generate([[1, 2, 3], [4, 5]], max_tokens=16, temperature=0.8, seed=7)

The option names are the reference's (``--max-tokens``, ``--temperature``, ``--top-k``,
``--top-p``, ``--seed``: src/main.rs:401-417, :956-990; the sampler's further options:
src/inference.rs:1716-1757). Prompts are token ids: tokenizers are outside this library.
"""
from __future__ import annotations

import json
import os

import torch

from .engine.generate import GenerationResult, generate as _generate
from .engine.model import DecoderModel, StepEntry, parse_dtype
from .sampling.options import SamplingOptions
from .sampling.sampler import Sampler


class LanguageModel:
    """A loaded model with a cache of its own for ``generate``."""

    def __init__(self, model: DecoderModel, stop_token_ids=()):
        self.model = model
        self.stop_token_ids = tuple(stop_token_ids)
        self._cache = None
        self._cache_tokens = 0

    @property
    def config(self):
        return self.model.typed_config

    def new_cache(self, max_tokens: int, max_slots: int | None = None):
        return self.model.new_cache(max_tokens, max_slots)

    def step(self, cache, entries) -> torch.Tensor:
        """``entries``: StepEntry(slot, tokens, want) or such tuples; see DecoderModel.step."""
        return self.model.step(cache, entries)

    def _cache_for(self, prompts, max_tokens, max_batch):
        per = list(max_tokens) if isinstance(max_tokens, (list, tuple)) else [max_tokens] * len(prompts)
        need = sorted((((len(p) + m + 63) // 64) * 64 for p, m in zip(prompts, per)), reverse=True)
        width = min(len(need), max_batch or len(need))
        tokens = max(64, sum(need[:width]))
        if self._cache is None or self._cache_tokens < tokens:
            if self._cache is not None:
                self.model.drop_graphs(self._cache)
            self._cache = None
            self._cache = self.model.new_cache(tokens)
            self._cache_tokens = tokens
        return self._cache

    def generate(self, prompts, max_tokens: int = 128, *, temperature: float = 0.0, top_k=None, top_p=None,
                 min_p=None, seed=None, presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                 repeat_penalty: float = 1.0, logit_bias=(), stop_token_ids=None, max_batch: int | None = None,
                 cache=None, details: bool = False, on_step=None):
        """Generate for a list of prompts (lists of token ids). Returns the generated ids per
        prompt (the stop token included), or ``GenerationResult`` objects with ``details``."""
        single = bool(prompts) and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        options = SamplingOptions(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, seed=seed,
                                  presence_penalty=presence_penalty, frequency_penalty=frequency_penalty,
                                  repeat_penalty=repeat_penalty, logit_bias=list(logit_bias))
        sampler = Sampler(options, self.model.vocab_size, self.model.device)
        stops = self.stop_token_ids if stop_token_ids is None else tuple(stop_token_ids)
        cache = cache if cache is not None else self._cache_for(prompts, max_tokens, max_batch)
        results = _generate(self.model, cache, sampler, prompts, max_tokens, stop_ids=stops, max_batch=max_batch,
                            on_step=on_step)
        sampler.check()
        self.model.check_device_errors()
        out = results if details else [r.tokens for r in results]
        return out[0] if single else out


def load(folder: str, dtype="bfloat16", device="cuda", options=None) -> LanguageModel:
    """Load ``folder`` (config.json, model.safetensors or shards). Stop tokens come from
    ``generation_config.json``'s ``eos_token_id`` if that file exists, else from config.json.
    ``options``: a ``KernelOptions`` (the defaults are the product path)."""
    model = DecoderModel.from_folder(folder, dtype=parse_dtype(dtype), device=device, options=options)
    stops = model.plan.stop_token_ids
    gen = os.path.join(folder, "generation_config.json")
    if os.path.isfile(gen):
        with open(gen) as f:
            e = json.load(f).get("eos_token_id")
        if e is not None:
            stops = tuple(e) if isinstance(e, list) else (int(e),)
    return LanguageModel(model, stops)


def from_random(config: dict, seed: int, dtype="bfloat16", device="cuda", options=None) -> LanguageModel:
    """A model of ``config`` (a config.json dict) with random weights drawn on the device:
    the same distributions as the random-weights folder, without the folder."""
    from .weights.random_init import random_tensors
    dt = parse_dtype(dtype)
    model = DecoderModel.from_config(config, dtype=dt, device=device, options=options)
    store = torch.bfloat16 if dt == torch.bfloat16 else torch.float32
    model.load_tensors(_DeviceRandom(model.tensor_specs(), seed, store, device))
    return LanguageModel(model, model.plan.stop_token_ids)


class _DeviceRandom:
    """Tensor source that draws each tensor on the device when it is asked for."""

    def __init__(self, specs, seed, dtype, device):
        self.specs, self.seed, self._dtype, self.device = specs, seed, dtype, device

    def names(self):
        return list(self.specs)

    def shape(self, name):
        return list(self.specs[name].shape)

    def dtype(self, name):
        return self._dtype

    def tensor(self, name):
        from .weights.random_init import random_tensor
        return random_tensor(name, self.specs[name], self.seed, self._dtype, self.device)
