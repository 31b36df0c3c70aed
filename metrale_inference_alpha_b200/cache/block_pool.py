"""Paged KV cache: fixed-size token blocks, a free list and per-block reference counts.

Layout per attention layer: K pool and V pool, each ``[num_blocks, block_size, kv_heads,
head_dim]`` in bf16 or e4m3 bytes (per-tensor dequant scales live beside the pools). MLA
layers keep one latent pool ``[num_blocks, block_size, 1, kv_lora + rope]``.
Role of the reference's ``crates/cache/src/kv_cache.rs`` (``KvCacheConfig`` block-byte math,
``PagedKvCache`` free list + refcounts) and ``model-engine/src/factory/build.rs`` (KV budget).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


class NoFreeBlocks(RuntimeError):
    """Raised when an allocation cannot be met; the scheduler answers by evicting prefix-cache
    blocks or preempting a sequence."""


@dataclass
class KvCacheConfig:
    num_layers: int                 # layers that own a KV pool
    kv_heads: int
    head_dim: int
    block_size: int = 16
    dtype: str = "bf16"             # bf16 | fp8
    v_head_dim: Optional[int] = None
    has_v: bool = True              # False for MLA latent caches
    high_precision_layers: tuple = ()   # cache layers kept in bf16 although dtype is fp8

    @property
    def elem_bytes(self) -> int:
        return 1 if self.dtype == "fp8" else 2

    def layer_dtype(self, i: int) -> str:
        return "bf16" if (self.dtype == "fp8" and i in self.high_precision_layers) else self.dtype

    def block_bytes(self) -> int:
        """Bytes one block occupies across all layers (K and V)."""
        per_elem = self.block_size * self.kv_heads * (self.head_dim + ((self.v_head_dim or self.head_dim) if self.has_v else 0))
        return sum(per_elem * (1 if self.layer_dtype(i) == "fp8" else 2) for i in range(self.num_layers))

    def blocks_for_budget(self, nbytes: int) -> int:
        return max(0, nbytes // max(1, self.block_bytes()))

    def blocks_for_tokens(self, tokens: int) -> int:
        return (tokens + self.block_size - 1) // self.block_size


class BlockAllocator:
    """Free list + reference counts. Block 0 is reserved as the "null" block padded rows and
    unused block-table entries point at, so a stray read never leaves the pool."""

    def __init__(self, num_blocks: int):
        assert num_blocks >= 2
        self.num_blocks = num_blocks
        self.refcount = [0] * num_blocks
        self.refcount[0] = 1 << 30
        self._free = list(range(num_blocks - 1, 0, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_blocks - 1 - len(self._free)

    def alloc(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise NoFreeBlocks(f"need {n} blocks, {len(self._free)} free")
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self.refcount[b] = 1
        return out

    def incref(self, blocks) -> None:
        for b in blocks:
            assert self.refcount[b] > 0, f"incref on free block {b}"
            self.refcount[b] += 1

    def free(self, blocks) -> List[int]:
        """Drop one reference per block; returns the blocks that became free."""
        released = []
        for b in blocks:
            if b == 0:
                continue
            assert self.refcount[b] > 0, f"double free of block {b}"
            self.refcount[b] -= 1
            if self.refcount[b] == 0:
                self._free.append(b)
                released.append(b)
        return released


class PagedKvCache:
    """Device pools + allocator. ``k[i]`` / ``v[i]`` index by *cache layer* (the i-th layer
    that owns a pool), see ``layer_map``."""

    def __init__(self, cfg: KvCacheConfig, num_blocks: int, device="cpu", poison: bool = False):
        self.cfg = cfg
        self.num_blocks = num_blocks
        self.device = torch.device(device)
        from . import make_allocator
        self.allocator = make_allocator(num_blocks)
        shape_k = (num_blocks, cfg.block_size, cfg.kv_heads, cfg.head_dim)
        shape_v = (num_blocks, cfg.block_size, cfg.kv_heads, cfg.v_head_dim or cfg.head_dim)
        fill = torch.full if poison else None
        self.k: List[torch.Tensor] = []
        self.v: List[Optional[torch.Tensor]] = []
        for li in range(cfg.num_layers):
            dt = torch.uint8 if cfg.layer_dtype(li) == "fp8" else torch.bfloat16
            if poison:
                # new blocks start as 0xFF bytes (NaN in bf16 / e4m3) so a read of a never
                # written slot shows up in the output (kv_poison in the reference)
                self.k.append(torch.full(shape_k, 255, dtype=torch.uint8, device=device).view(dt)
                              if dt == torch.uint8 else
                              torch.full(shape_k, float("nan"), dtype=dt, device=device))
                self.v.append(None if not cfg.has_v else
                              (torch.full(shape_v, 255, dtype=torch.uint8, device=device)
                               if dt == torch.uint8 else torch.full(shape_v, float("nan"), dtype=dt, device=device)))
            else:
                from ..utils.alloc_ledger import ledger
                self.k.append(ledger().alloc(shape_k, dt, device, "kv pool (k)"))
                self.v.append(ledger().alloc(shape_v, dt, device, "kv pool (v)") if cfg.has_v else None)
        del fill
        # dequant multipliers (stored value = amax / 448); 1.0 until calibrated or loaded
        self.k_scale = [torch.ones(1, dtype=torch.float32, device=device) for _ in range(cfg.num_layers)]
        self.v_scale = [torch.ones(1, dtype=torch.float32, device=device) for _ in range(cfg.num_layers)]

    def bytes(self) -> int:
        return self.cfg.block_bytes() * self.num_blocks

    def copy_block(self, src: int, dst: int) -> None:
        """Copy-on-write support for a shared, partially filled last block."""
        for i in range(self.cfg.num_layers):
            self.k[i][dst].copy_(self.k[i][src])
            if self.v[i] is not None:
                self.v[i][dst].copy_(self.v[i][src])

    # ---- sequence spill / restore (crates/cache/src/kv_spill.rs)
    def gather_blocks(self, blocks: List[int]) -> Dict[str, torch.Tensor]:
        idx = torch.tensor(blocks, dtype=torch.long, device=self.device)
        out = {}
        for i in range(self.cfg.num_layers):
            out[f"k{i}"] = self.k[i][idx].cpu()
            if self.v[i] is not None:
                out[f"v{i}"] = self.v[i][idx].cpu()
        return out

    def scatter_blocks(self, blocks: List[int], data: Dict[str, torch.Tensor]) -> None:
        idx = torch.tensor(blocks, dtype=torch.long, device=self.device)
        for i in range(self.cfg.num_layers):
            self.k[i][idx] = data[f"k{i}"].to(self.device)
            if self.v[i] is not None:
                self.v[i][idx] = data[f"v{i}"].to(self.device)
