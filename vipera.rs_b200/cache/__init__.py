"""The cache: native bookkeeping of pages and state slots, and the device memory they index."""
from .pools import CacheGroup, CachePools, plan_groups

__all__ = ["CacheGroup", "CachePools", "plan_groups"]
