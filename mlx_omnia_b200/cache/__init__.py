"""Paged key/value cache, block tables and per-request state slots."""

from mlx_omnia_b200.cache.manager import CacheError, CacheManager, PagePool, RequestCache

__all__ = ["CacheError", "CacheManager", "PagePool", "RequestCache"]
