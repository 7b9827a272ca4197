"""Greedy and temperature / min_p / top-k / top-p sampling, with repetition, presence and frequency penalties, added logits,
the no-repeat-n-gram rule and the stop on a repeating pattern."""

from .defaults import card_sampling, resolve as resolve_filters
from .sampler import NoRepeatIndex, Sampler, SampleRow, SamplingParams, repeating_pattern

__all__ = ["NoRepeatIndex", "Sampler", "SampleRow", "SamplingParams", "card_sampling", "repeating_pattern", "resolve_filters"]
