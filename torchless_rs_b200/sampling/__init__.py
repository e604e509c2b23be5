from .params import SamplingParams, uniform_for

__all__ = ["SamplingParams", "uniform_for", "Sampler"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
