from .block_pool import BlockAllocator, KvCacheConfig, PagedKvCache, NoFreeBlocks  # noqa: F401
from .radix import RadixTree, PrefixMatch  # noqa: F401
from .state_pool import StatePool  # noqa: F401
