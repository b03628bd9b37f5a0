from .params import SamplingParams, XorShift64, penalty_window

__all__ = ["SamplingParams", "XorShift64", "penalty_window", "Sampler"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
