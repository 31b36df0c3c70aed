"""Storage tiers below device memory: KV blocks in files attended tile by tile (``high_speed_swap``),
MoE expert records paged into a device arena (``expert_store``), a file-backed row cache for large
embedding tables (``row_cache``), the byte stores under them (``backend``) and a capability probe
(``probe``). Reference: ``crates/storage``."""
from .backend import CascadeBackend, CommitLedger, FileBackend, KvLayout, MemoryBackend  # noqa: F401
from .high_speed_swap import HighSpeedSwap, HighSpeedSwapConfig, ModelDims, ResidentTail  # noqa: F401
