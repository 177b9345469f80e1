from .params import PENALTY_WINDOW, SamplingParams
from .sampler import Sampler, uniform_for

__all__ = ["PENALTY_WINDOW", "SamplingParams", "Sampler", "uniform_for"]
