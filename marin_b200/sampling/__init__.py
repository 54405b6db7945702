"""Greedy, temperature, top-k and top-p sampling."""
from .sampler import Sampler, SamplerError, SamplingParams, best_index

__all__ = ["Sampler", "SamplerError", "SamplingParams", "best_index"]
