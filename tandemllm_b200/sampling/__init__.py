"""Greedy and temperature / min_p / top-k / top-p sampling, with repetition, presence and frequency penalties and added logits."""

from .sampler import Sampler, SampleRow, SamplingParams

__all__ = ["Sampler", "SampleRow", "SamplingParams"]
