from .llama import LlamaConfig, RopeScaling
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from .registry import (Architecture, architecture_of, known_architectures, llama_plan, load_config,
                       read_config_json, register_architecture)

__all__ = ["LlamaConfig", "RopeScaling", "LayerSpec", "ModelPlan", "PartSpec", "ScheduleEntry", "Architecture",
           "architecture_of", "known_architectures", "llama_plan", "load_config", "read_config_json",
           "register_architecture"]
