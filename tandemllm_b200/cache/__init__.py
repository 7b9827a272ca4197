"""Paged keys and values with block tables, and per-request state slots."""

from .manager import CacheManager, OutOfPages, PageGroup, PagePool

__all__ = ["CacheManager", "OutOfPages", "PageGroup", "PagePool"]
