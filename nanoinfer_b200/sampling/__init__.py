from .params import SamplingParams
from .sampler import SampleRow, Sampler, uniform_for

__all__ = ["SamplingParams", "SampleRow", "Sampler", "uniform_for"]
