from .sampler import Sampler, SamplingRow

__all__ = ["Sampler", "SamplingRow"]
