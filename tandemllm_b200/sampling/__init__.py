"""Greedy and temperature / min_p / top-k / top-p sampling."""

from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]
