from atomserve_b200.cache.block_allocator import BlockAllocator, OutOfBlocksError, block_hash, blocks_for_tokens
from atomserve_b200.cache.manager import CacheGroup, CacheManager, RequestCache
from atomserve_b200.cache.state_slots import StateSlots

__all__ = [
    "BlockAllocator", "CacheGroup", "CacheManager", "OutOfBlocksError", "RequestCache",
    "StateSlots", "block_hash", "blocks_for_tokens",
]  # fmt: skip
