from .sampler import Sampler, SamplingParams, request_seed, uniform_draw

__all__ = ["Sampler", "SamplingParams", "request_seed", "uniform_draw"]
