from .block_pool import BlockAllocator, KvCacheConfig, PagedKvCache, NoFreeBlocks  # noqa: F401
from .radix import RadixTree, PrefixMatch  # noqa: F401
from .state_pool import StatePool  # noqa: F401


def make_allocator(num_blocks: int):
    """The C++ allocator when the host runtime library is built, else the Python one."""
    from .. import native
    if native.available():
        return native.NativeBlockAllocator(num_blocks)
    return BlockAllocator(num_blocks)


def make_radix(allocator, block_size: int, needs_snapshot: bool = False, on_snapshot_evict=None):
    """Prefix index matching the allocator's implementation (they share the refcounts)."""
    from .. import native
    if native.available() and isinstance(allocator, native.NativeBlockAllocator):
        return native.NativeRadixTree(allocator, block_size, needs_snapshot, on_snapshot_evict)
    return RadixTree(allocator, block_size, needs_snapshot, on_snapshot_evict)
