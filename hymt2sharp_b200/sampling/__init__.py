from .params import GREEDY, SamplingParams
from .sampler import BatchSampler

__all__ = ["GREEDY", "SamplingParams", "BatchSampler"]
