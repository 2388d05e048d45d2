"""Paged key/value cache, block tables, and per-request state slots."""

from .manager import CacheError, CacheGroup, CacheManager, PagePool
from .spec import HeadRowPagesSpec, KVPagesSpec, PagesSpec, StateSpec, TokenPagesSpec

__all__ = ["CacheError", "CacheGroup", "CacheManager", "PagePool", "HeadRowPagesSpec", "KVPagesSpec", "PagesSpec", "StateSpec", "TokenPagesSpec"]
