"""Byte stores of the KV storage tier.

``KvLayout``      geometry of one layer file: block ``b`` occupies ``block_bytes`` contiguous bytes
                  at ``b * block_bytes`` (the K stripes of every kv head, then the V stripes; each
                  stripe = one *group* of ``block_size x head_dim`` elements padded to the filesystem
                  block), one pre-allocated file ``layer_00000.kv`` per layer.
``FileBackend``   reads / writes whole blocks with positional I/O from a small thread pool (the calls
                  release the GIL, so several NVMe requests are in flight), optionally ``O_DIRECT``
                  through page-aligned pinned buffers.
``MemoryBackend`` the same interface over host tensors (tests, and machines without a scratch disk).
``CascadeBackend`` a write-back cache of blocks in pinned host memory (tier 1) in front of another
                  backend: writes land in tier 1, the least recently used block is written down when it
                  is full, reads are served from tier 1 on a hit and forwarded on a miss (misses are
                  not promoted).
``CommitLedger``  running total of reserved bytes against a ceiling (shared by servers that hand out
                  memory to peers).

Reference: ``crates/storage/src/{layout,group,backend/*,cascade_backend,cascade_policy,blade_cap}.rs``.
"""
from __future__ import annotations

import concurrent.futures as cf
import mmap
import os
import threading
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass(frozen=True)
class KvLayout:
    num_layers: int
    num_blocks: int           # blocks per layer file
    block_size: int           # tokens
    kv_heads: int
    head_dim: int
    elem_bytes: int = 2
    fs_block: int = 4096

    def __post_init__(self):
        for name in ("num_layers", "num_blocks", "block_size", "kv_heads", "head_dim", "elem_bytes"):
            if getattr(self, name) <= 0:
                raise ValueError(f"KvLayout.{name} must be positive")
        if self.fs_block <= 0 or self.fs_block & (self.fs_block - 1):
            raise ValueError("fs_block must be a power of two")

    @property
    def group_payload(self) -> int:
        return self.block_size * self.head_dim * self.elem_bytes

    @property
    def group_stride(self) -> int:
        return _round_up(self.group_payload, self.fs_block)

    @property
    def block_bytes(self) -> int:
        return 2 * self.kv_heads * self.group_stride

    @property
    def bytes_per_layer(self) -> int:
        return self.num_blocks * self.block_bytes

    def file_offset(self, block: int, kind: int = 0, kv_head: int = 0) -> int:
        """Byte offset of a group (kind 0 = K, 1 = V) inside its layer file."""
        if not (0 <= block < self.num_blocks and kind in (0, 1) and 0 <= kv_head < self.kv_heads):
            raise IndexError(f"group ({block}, {kind}, {kv_head}) outside the layout")
        return block * self.block_bytes + (kind * self.kv_heads + kv_head) * self.group_stride

    def group_id(self, layer: int, block: int, kind: int, kv_head: int) -> int:
        """Dense id in the same order as (layer, file_offset)."""
        if not 0 <= layer < self.num_layers:
            raise IndexError("layer outside the layout")
        self.file_offset(block, kind, kv_head)
        return ((layer * self.num_blocks + block) * 2 + kind) * self.kv_heads + kv_head

    def layer_path(self, root: str, layer: int) -> str:
        return os.path.join(root, f"layer_{layer:05d}.kv")


class CommitLedger:
    """``reserve(n)`` succeeds while the total stays under the cap (0 = no cap); the returned handle
    gives the bytes back on ``release()`` (idempotent)."""

    class Reservation:
        def __init__(self, ledger, n):
            self._ledger, self.bytes = ledger, n

        def release(self):
            if self._ledger is not None:
                with self._ledger._lock:
                    self._ledger.committed -= self.bytes
                self._ledger = None

        __del__ = release

    def __init__(self, cap_bytes: int = 0):
        self.cap, self.committed = cap_bytes, 0
        self._lock = threading.Lock()

    def reserve(self, n: int) -> Optional["CommitLedger.Reservation"]:
        if n < 0:
            raise ValueError("negative reservation")
        with self._lock:
            if self.cap and self.committed + n > self.cap:
                return None
            self.committed += n
        return CommitLedger.Reservation(self, n)


def pinned_bytes(n: int) -> torch.Tensor:
    """Page-aligned host buffer of ``n`` bytes, pinned when a CUDA device is present."""
    buf = torch.empty(n + 4096, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
    off = (-buf.data_ptr()) % 4096
    return buf[off:off + n]


class StorageBackend:
    """Block-granular interface every tier implements. Buffers are uint8 host tensors of
    ``layout.block_bytes`` bytes (page-aligned for O_DIRECT)."""

    layout: KvLayout

    def write_block(self, layer: int, block: int, buf: torch.Tensor) -> None:
        raise NotImplementedError

    def read_block(self, layer: int, block: int, buf: torch.Tensor) -> None:
        raise NotImplementedError

    def read_blocks_async(self, layer: int, blocks: List[int], bufs: List[torch.Tensor]) -> List[cf.Future]:
        done = []
        for b, buf in zip(blocks, bufs):
            f: cf.Future = cf.Future()
            try:
                self.read_block(layer, b, buf)
                f.set_result(None)
            except Exception as e:          # surfaced by the caller's .result()
                f.set_exception(e)
            done.append(f)
        return done

    def flush(self) -> None:
        pass

    def close(self) -> None:
        pass


class MemoryBackend(StorageBackend):
    def __init__(self, layout: KvLayout):
        self.layout = layout
        self._blocks: Dict[Tuple[int, int], torch.Tensor] = {}
        self.stats = {"reads": 0, "writes": 0}

    def write_block(self, layer, block, buf):
        self.layout.file_offset(block)
        self._blocks[(layer, block)] = buf[: self.layout.block_bytes].clone()
        self.stats["writes"] += 1

    def read_block(self, layer, block, buf):
        src = self._blocks.get((layer, block))
        if src is None:
            raise KeyError(f"block ({layer}, {block}) was never written")
        buf[: self.layout.block_bytes].copy_(src)
        self.stats["reads"] += 1


class FileBackend(StorageBackend):
    def __init__(self, root: str, layout: KvLayout, *, create: bool = True, direct: bool = False, workers: int = 8):
        self.layout, self.root = layout, root
        self.direct = bool(direct and hasattr(os, "O_DIRECT"))
        os.makedirs(root, exist_ok=True)
        self._fds: List[int] = []
        for layer in range(layout.num_layers):
            path = layout.layer_path(root, layer)
            if not create and not os.path.exists(path):
                raise FileNotFoundError(path)
            flags = os.O_RDWR | (os.O_CREAT if create else 0) | (os.O_DIRECT if self.direct else 0)
            try:
                fd = os.open(path, flags, 0o600)
            except OSError:
                if not self.direct:
                    raise
                self.direct = False          # tmpfs and some overlay filesystems refuse O_DIRECT
                fd = os.open(path, os.O_RDWR | (os.O_CREAT if create else 0), 0o600)
            if os.fstat(fd).st_size < layout.bytes_per_layer:
                if not create:
                    os.close(fd)
                    raise ValueError(f"{path} is shorter than the layout ({layout.bytes_per_layer} bytes)")
                try:
                    os.posix_fallocate(fd, 0, layout.bytes_per_layer)
                except OSError:
                    os.ftruncate(fd, layout.bytes_per_layer)
            self._fds.append(fd)
        self._pool = cf.ThreadPoolExecutor(max_workers=workers, thread_name_prefix="kvtier-io")
        self.stats = {"reads": 0, "writes": 0, "bytes_in": 0, "bytes_out": 0}

    def _view(self, buf: torch.Tensor) -> memoryview:
        n = self.layout.block_bytes
        if buf.dtype != torch.uint8 or buf.numel() < n or not buf.is_contiguous() or buf.is_cuda:
            raise ValueError("buffer must be a contiguous uint8 host tensor of block_bytes")
        if self.direct and buf.data_ptr() % mmap.PAGESIZE:
            raise ValueError("O_DIRECT needs a page-aligned buffer (use pinned_bytes)")
        return memoryview(buf[:n].numpy())

    def write_block(self, layer, block, buf):
        off = self.layout.file_offset(block)
        n = os.pwritev(self._fds[layer], [self._view(buf)], off)
        if n != self.layout.block_bytes:
            raise IOError(f"short write: {n} of {self.layout.block_bytes} bytes")
        self.stats["writes"] += 1
        self.stats["bytes_out"] += n

    def read_block(self, layer, block, buf):
        off = self.layout.file_offset(block)
        n = os.preadv(self._fds[layer], [self._view(buf)], off)
        if n != self.layout.block_bytes:
            raise IOError(f"short read: {n} of {self.layout.block_bytes} bytes")
        self.stats["reads"] += 1
        self.stats["bytes_in"] += n

    def read_blocks_async(self, layer, blocks, bufs):
        return [self._pool.submit(self.read_block, layer, b, buf) for b, buf in zip(blocks, bufs)]

    def flush(self):
        for fd in self._fds:
            os.fsync(fd)

    def close(self):
        self._pool.shutdown(wait=True)
        for fd in self._fds:
            os.close(fd)
        self._fds = []


class CascadeBackend(StorageBackend):
    def __init__(self, backing: StorageBackend, slots: int):
        if slots <= 0:
            raise ValueError("tier 1 needs at least one slot")
        self.layout, self.backing = backing.layout, backing
        self._arena = pinned_bytes(slots * self.layout.block_bytes).view(slots, self.layout.block_bytes)
        self._free = list(range(slots - 1, -1, -1))
        self._lru: "OrderedDict[Tuple[int, int], int]" = OrderedDict()      # key -> slot, oldest first
        self._dirty: set = set()
        self.stats = {"hits": 0, "misses": 0, "writebacks": 0}

    def _slot_for(self, key) -> int:
        if key in self._lru:
            self._lru.move_to_end(key)
            return self._lru[key]
        if not self._free:
            old, slot = self._lru.popitem(last=False)
            if old in self._dirty:
                self.backing.write_block(old[0], old[1], self._arena[slot])
                self._dirty.discard(old)
                self.stats["writebacks"] += 1
            self._free.append(slot)
        slot = self._free.pop()
        self._lru[key] = slot
        return slot

    def write_block(self, layer, block, buf):
        key = (layer, block)
        self._arena[self._slot_for(key)].copy_(buf[: self.layout.block_bytes])
        self._dirty.add(key)

    def read_block(self, layer, block, buf):
        key = (layer, block)
        slot = self._lru.get(key)
        if slot is not None:
            self._lru.move_to_end(key)
            buf[: self.layout.block_bytes].copy_(self._arena[slot])
            self.stats["hits"] += 1
        else:
            self.backing.read_block(layer, block, buf)
            self.stats["misses"] += 1

    def read_blocks_async(self, layer, blocks, bufs):
        out: List[cf.Future] = []
        miss_b, miss_buf, miss_at = [], [], []
        for i, (b, buf) in enumerate(zip(blocks, bufs)):
            if (layer, b) in self._lru:
                f: cf.Future = cf.Future()
                self.read_block(layer, b, buf)
                f.set_result(None)
                out.append(f)
            else:
                out.append(None)
                miss_b.append(b)
                miss_buf.append(buf)
                miss_at.append(i)
                self.stats["misses"] += 1
        for i, f in zip(miss_at, self.backing.read_blocks_async(layer, miss_b, miss_buf)):
            out[i] = f
        return out

    def flush(self):
        for key in sorted(self._dirty):
            self.backing.write_block(key[0], key[1], self._arena[self._lru[key]])
            self.stats["writebacks"] += 1
        self._dirty.clear()
        self.backing.flush()

    def close(self):
        self.flush()
        self.backing.close()
