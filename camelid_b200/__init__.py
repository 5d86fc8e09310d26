"""camelid_b200: a small generation library for the dense Llama decoder on one B200.

Importing the package needs no GPU; running a step does (the CUDA kernels are compiled at
their first use and there is no other path)."""
from .config import LlamaConfig, load_config, register_architecture
from .errors import (CacheError, CamelidError, ConfigError, KernelError, SafetensorsError, SamplingError, StepError,
                     UnknownArchitectureError, WeightsError)

__version__ = "0.1.0"
__all__ = ["LlamaConfig", "load_config", "register_architecture", "load", "from_random", "LanguageModel",
           "DecoderModel", "StepEntry", "SamplingOptions", "KernelOptions", "write_random_model", "memory_plan", "MemoryPlan", "MemoryBudgetError",
           "CacheError", "CamelidError", "ConfigError", "KernelError", "SafetensorsError", "SamplingError",
           "StepError", "UnknownArchitectureError", "WeightsError"]

_LAZY = {
    "load": ("camelid_b200.api", "load"), "from_random": ("camelid_b200.api", "from_random"),
    "LanguageModel": ("camelid_b200.api", "LanguageModel"),
    "DecoderModel": ("camelid_b200.engine.model", "DecoderModel"),
    "StepEntry": ("camelid_b200.engine.model", "StepEntry"),
    "SamplingOptions": ("camelid_b200.sampling.options", "SamplingOptions"),
    "KernelOptions": ("camelid_b200.options", "KernelOptions"),
    "memory_plan": ("camelid_b200.memory", "memory_plan"),
    "MemoryPlan": ("camelid_b200.memory", "MemoryPlan"),
    "MemoryBudgetError": ("camelid_b200.memory", "MemoryBudgetError"),
    "write_random_model": ("camelid_b200.weights.random_init", "write_random_model"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)
