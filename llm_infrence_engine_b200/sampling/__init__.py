from .sampler import Sampler, SamplingParams, uniform_from

__all__ = ["Sampler", "SamplingParams", "uniform_from"]
