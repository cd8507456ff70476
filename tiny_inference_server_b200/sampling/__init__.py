from .params import SamplingParams
from .sampler import Sampler, SampleSpec

__all__ = ["SamplingParams", "Sampler", "SampleSpec"]
