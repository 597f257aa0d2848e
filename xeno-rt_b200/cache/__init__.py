"""The cache: a slot for each sequence, block storage for keys and values of each layer, fixed-size
state per sequence, and the allocators behind them."""
from .spec import KVNeed, StateNeed
from .allocator import BlockAllocator, SlotAllocator
from .cache import Cache, KVStore, StateStore, BLOCK_TOKENS

__all__ = ["KVNeed", "StateNeed", "BlockAllocator", "SlotAllocator", "Cache", "KVStore", "StateStore",
           "BLOCK_TOKENS"]
