from .params import RECENT_TOKENS_WINDOW, SamplingParams
from .sampler import Sampler

__all__ = ["RECENT_TOKENS_WINDOW", "SamplingParams", "Sampler"]
