from .loader import check_tensors
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import ModelFiles, SafetensorsFile, write_safetensors

__all__ = ["check_tensors", "random_tensor", "random_tensors", "write_random_model", "ModelFiles", "SafetensorsFile",
           "write_safetensors"]
