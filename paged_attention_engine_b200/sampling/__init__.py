from .sampler import SamplingRow

__all__ = ["SamplingRow"]
