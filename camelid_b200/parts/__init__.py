from .base import Part, TensorSpec, build_block, build_part, known_parts, register_part
from . import norm, position, attention, feedforward, embedding, block  # noqa: F401  (registers the parts)

__all__ = ["Part", "TensorSpec", "build_block", "build_part", "known_parts", "register_part"]
