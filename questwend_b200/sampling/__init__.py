from .params import SamplingParams, GREEDY
from .sampler import DeviceSampler, PenaltyWindow

__all__ = ["SamplingParams", "GREEDY", "DeviceSampler", "PenaltyWindow"]
