from .params import SamplingParams
from .sampler import SampleHandle, Sampler, request_rng

__all__ = ["SamplingParams", "SampleHandle", "Sampler", "request_rng"]
