from .params import SamplingParams
from .sampler import Sampler, request_rng

__all__ = ["SamplingParams", "Sampler", "request_rng"]
