from .manager import CacheManager, GroupNeed, PagePool, OutOfPages, OutOfSlots
from .storage import allocate_caches, allocate_states, cache_bytes_per_token
