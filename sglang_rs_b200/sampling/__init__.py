from .params import SamplingParams
from .sampler import RequestRandom, Sampler, apply_penalties

__all__ = ["SamplingParams", "RequestRandom", "Sampler", "apply_penalties"]
