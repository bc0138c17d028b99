from .params import SamplingParams
from .rng import Xoshiro256
from .sampler import Sampler, greedy_token

__all__ = ["SamplingParams", "Xoshiro256", "Sampler", "greedy_token"]
