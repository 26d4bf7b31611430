"""Sequence slots, paged key/value storage per layer group, fixed-size per-sequence state."""

from .allocator import CacheError, IndexAllocator
from .cache import PAGE, Cache, KVGroup, KVRequest, LayerCache, SharedRequest, StateGroup, StateRequest

__all__ = ["CacheError", "IndexAllocator", "PAGE", "Cache", "KVGroup", "KVRequest", "LayerCache", "SharedRequest",
           "StateGroup", "StateRequest"]
