"""File-backed row cache for embedding tables that are larger than the memory set aside for them
(n-gram embedding tables of several hundred GB): rows fault from the checkpoint file into an arena
of ``slots`` rows, and the gather reads the arena by slot.

``resolve(ids)`` maps each row id of a batch to its arena slot (reading misses from the file) and
returns the slot indices; ``gather(ids)`` returns the rows themselves. A slot pinned since the last
``end_batch`` is never chosen as a victim; eviction is CLOCK (second chance) over the unpinned slots.
The invariant ``map[id] == s  <=>  slot_row[s] == id`` holds on every path out of ``resolve``,
including the error paths (a failed read leaves the slot empty). Files opened ``O_DIRECT`` are read in
4 KiB blocks through an aligned bounce buffer (one or two blocks cover a row).

Reference: ``crates/storage/src/ngram_cache.rs``, ``ngram_cache_fault.rs``.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from .backend import pinned_bytes


class RowCache:
    def __init__(self, path: str, *, num_rows: int, row_bytes: int, slots: int, dtype=torch.bfloat16,
                 file_offset: int = 0, device="cpu", direct: bool = False):
        if slots <= 0 or row_bytes <= 0 or num_rows <= 0:
            raise ValueError("slots, row_bytes and num_rows must be positive")
        self.num_rows, self.row_bytes, self.slots, self.base = num_rows, row_bytes, slots, file_offset
        self.direct = bool(direct and hasattr(os, "O_DIRECT"))
        try:
            self._fd = os.open(path, os.O_RDONLY | (os.O_DIRECT if self.direct else 0))
        except OSError:
            if not self.direct:
                raise
            self.direct = False
            self._fd = os.open(path, os.O_RDONLY)
        if os.fstat(self._fd).st_size < file_offset + num_rows * row_bytes:
            os.close(self._fd)
            raise ValueError("the file is shorter than the table")
        self.dtype = dtype
        self.device = torch.device(device)
        self.arena = torch.zeros(slots, row_bytes, dtype=torch.uint8, device=self.device)
        self.map: Dict[int, int] = {}
        self.slot_row: List[Optional[int]] = [None] * slots
        self.ref_bit = [False] * slots
        self.pinned = [False] * slots
        self.hand = 0
        self._bounce = pinned_bytes(2 * 4096 + ((row_bytes + 4095) // 4096) * 4096)
        self.stats = {"hits": 0, "misses": 0, "evictions": 0, "read_errors": 0}

    def table(self) -> torch.Tensor:
        """The arena as rows of ``dtype`` (what a gather kernel indexes by slot)."""
        return self.arena.view(self.dtype)

    def _read_row(self, row: int) -> torch.Tensor:
        off = self.base + row * self.row_bytes
        if self.direct:
            lo = off // 4096 * 4096
            n = (off + self.row_bytes + 4095) // 4096 * 4096 - lo
        else:
            lo, n = off, self.row_bytes
        got = os.preadv(self._fd, [memoryview(self._bounce[:n].numpy())], lo)
        if got < off - lo + self.row_bytes:
            raise IOError(f"short read of row {row}")
        return self._bounce[off - lo:off - lo + self.row_bytes]

    def _victim(self) -> int:
        for _ in range(2 * self.slots + 1):
            s = self.hand
            self.hand = (self.hand + 1) % self.slots
            if self.pinned[s]:
                continue
            if self.slot_row[s] is None:
                return s
            if self.ref_bit[s]:
                self.ref_bit[s] = False
                continue
            del self.map[self.slot_row[s]]
            self.slot_row[s] = None
            self.stats["evictions"] += 1
            return s
        raise MemoryError("every slot is pinned by the current batch: the arena is smaller than one batch's distinct rows")

    def resolve(self, ids: Sequence[int]) -> torch.Tensor:
        out = []
        for i in ids:
            i = int(i)
            if not 0 <= i < self.num_rows:
                raise IndexError(f"row {i} outside the table")
            s = self.map.get(i)
            if s is None:
                s = self._victim()
                try:
                    row = self._read_row(i)
                except Exception:
                    self.stats["read_errors"] += 1
                    raise                      # the slot stays empty: map and slot_row still agree
                self.arena[s].copy_(row)
                self.map[i], self.slot_row[s] = s, i
                self.stats["misses"] += 1
            else:
                self.stats["hits"] += 1
            self.ref_bit[s] = True
            self.pinned[s] = True
            out.append(s)
        return torch.tensor(out, dtype=torch.int64, device=self.device)

    def end_batch(self) -> None:
        self.pinned = [False] * self.slots

    def gather(self, ids: Sequence[int]) -> torch.Tensor:
        rows = self.table()[self.resolve(ids)]
        self.end_batch()
        return rows

    def check_invariant(self) -> bool:
        return (all(self.slot_row[s] == i for i, s in self.map.items())
                and all(r is None or self.map.get(r) == s for s, r in enumerate(self.slot_row)))

    def close(self) -> None:
        if self._fd >= 0:
            os.close(self._fd)
            self._fd = -1
