from .allocator import CacheError, IndexPool
from .cache import CachePlan, KVView, SequenceCache, StateView, plan_cache
from .needs import KVNeed, StateNeed

__all__ = ["CacheError", "IndexPool", "CachePlan", "KVView", "SequenceCache", "StateView", "plan_cache",
           "KVNeed", "StateNeed"]
