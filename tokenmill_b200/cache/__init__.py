from .allocator import OutOfPages, PageAllocator
from .manager import AllocStatus, CacheHandle, CacheManager, StateSlots, chain_hash

__all__ = ["OutOfPages", "PageAllocator", "AllocStatus", "CacheHandle", "CacheManager", "StateSlots", "chain_hash"]
