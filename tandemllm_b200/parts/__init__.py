"""Layers put together from parts: mixers, feed-forwards, norms, position encodings, arrangements."""

from . import attention, block, feed_forward, norm, position, short_conv  # noqa: F401  (each registers its kinds)
from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, PagedNeed, PagedSiteCache, Part,
                   Runtime, SlotNeed, SlotSiteCache, StepContext, make_part, register_part)
from .block import Layer
from .model import DecoderModel

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "PagedNeed", "PagedSiteCache",
           "Part", "Runtime", "SlotNeed", "SlotSiteCache", "StepContext", "make_part", "register_part", "Layer",
           "DecoderModel"]
