from .sampler import Sampler, uniform

__all__ = ["Sampler", "uniform"]
