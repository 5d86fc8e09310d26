from .options import SamplingOptions, splitmix64, unit_draw

__all__ = ["SamplingOptions", "splitmix64", "unit_draw", "Sampler"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
