from .allocator import PAGE_TOKENS, CacheError, CacheLedger, pages_for  # noqa: F401
from .kv import CacheGroup, CacheView, KVCache, KVRequest, StateRequest  # noqa: F401
