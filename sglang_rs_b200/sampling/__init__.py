from .params import SamplingParams
from .sampler import RequestRandom, Sampler, SeenCounts

__all__ = ["SamplingParams", "RequestRandom", "Sampler", "SeenCounts"]
