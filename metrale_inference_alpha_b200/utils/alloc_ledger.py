"""Ledger of the engine's long-lived device allocations, with optional red zones.

Every pool the engine allocates once (KV pools, recurrent-state pool, kernel workspaces, staging
buffers, graph-static tensors) goes through ``alloc``: the ledger records its size and the allocating
call site, so "where did the memory go" is a table (``report``) instead of a guess, and the gap between
the ledger's total and what the caching allocator reserved (``slack``) shows what small transient
allocations and fragmentation hold.

Red zones (``METRALE_REDZONE=<bytes>``, off by default): every ledger allocation gets a guard band of
that many bytes behind it, filled with a fixed pattern; ``check`` compares all bands on the device
(one reduction per band, no copy of the band) and names the allocations whose band was overwritten —
an out-of-bounds write by a kernel shows up at the next check, attributed to the buffer it ran past,
instead of as corrupted output much later. ``METRALE_REDZONE_EVERY=<n>`` makes the engine check every
n-th step. ``refill`` restores the pattern after a report.

Reference: ``crates/gpu-runtime/src/cuda_backend/{alloc_ledger,redzone}.rs``.
"""
from __future__ import annotations

import os
import sys
import threading
import weakref
from collections import deque
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

PATTERN = 0xA5


@dataclass
class Entry:
    name: str
    site: str
    nbytes: int
    device: str
    guard: Optional[torch.Tensor] = None      # the band behind the allocation (uint8)


def _call_site(depth: int = 2) -> str:
    f = sys._getframe(depth)
    return f"{os.path.basename(f.f_code.co_filename)}:{f.f_lineno}"


class AllocLedger:
    def __init__(self, redzone_bytes: Optional[int] = None):
        if redzone_bytes is None:
            redzone_bytes = int(os.environ.get("METRALE_REDZONE", "0") or 0)
        if redzone_bytes < 0 or redzone_bytes % 16:
            raise ValueError("the red zone must be a non-negative multiple of 16 bytes")
        self.redzone = redzone_bytes
        self._live: Dict[int, Entry] = {}
        self._next = 0
        self._lock = threading.Lock()
        self._dead: "deque[int]" = deque()           # keys of tensors that died; taken out of _live under the lock

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape, dtype=torch.uint8, device="cpu", name: str = "", fill: Optional[float] = 0, site: Optional[str] = None
              ) -> torch.Tensor:
        """A tensor of ``shape`` recorded under ``name``; with red zones on it is the front part of a
        larger byte buffer whose tail is the guard band. The entry disappears when the tensor dies."""
        site = site or _call_site()
        shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        n = 1
        for s in shape:
            n *= int(s)
        elem = torch.empty((), dtype=dtype).element_size()
        nbytes = n * elem
        guard = None
        if self.redzone:
            pad = (-nbytes) % 16
            raw = torch.empty(nbytes + pad + self.redzone, dtype=torch.uint8, device=device)
            guard = raw[nbytes + pad:]
            guard.fill_(PATTERN)
            t = raw[:nbytes].view(dtype).view(shape)
        else:
            t = torch.empty(shape, dtype=dtype, device=device)
        if fill is not None:
            t.fill_(fill) if fill else t.zero_()
        with self._lock:
            self._reap()
            key = self._next
            self._next += 1
            self._live[key] = Entry(name or site, site, nbytes, str(t.device), guard)
        weakref.finalize(t, self._drop, key)
        return t

    def track(self, t: torch.Tensor, name: str, site: Optional[str] = None) -> torch.Tensor:
        """Record an allocation made elsewhere (no red zone can be added after the fact)."""
        with self._lock:
            self._reap()
            key = self._next
            self._next += 1
            self._live[key] = Entry(name, site or _call_site(), t.numel() * t.element_size(), str(t.device))
        weakref.finalize(t, self._drop, key)
        return t

    def _drop(self, key: int) -> None:
        # A tensor's finalizer runs wherever the garbage collector happens to run: that can be inside one of this
        # ledger's own locked sections (creating an Entry allocates), on the very thread that holds the lock. It
        # therefore takes no lock and touches no dict: it leaves the key in a queue that the locked sections drain.
        self._dead.append(key)

    def _reap(self) -> None:
        """Forget the entries of dead tensors. The caller holds the lock."""
        while self._dead:
            self._live.pop(self._dead.popleft(), None)

    # ------------------------------------------------------------------ reports
    def total_bytes(self, device: Optional[str] = None) -> int:
        with self._lock:
            self._reap()
            return sum(e.nbytes + (e.guard.numel() if e.guard is not None else 0) for e in self._live.values()
                       if device is None or e.device == device)

    def report(self) -> List[dict]:
        """Live allocations grouped by name, largest first."""
        groups: Dict[Tuple[str, str], List[int]] = {}
        sites: Dict[Tuple[str, str], str] = {}
        with self._lock:
            self._reap()
            for e in self._live.values():
                groups.setdefault((e.name, e.device), []).append(e.nbytes)
                sites.setdefault((e.name, e.device), e.site)
        rows = [{"name": k[0], "site": sites[k], "device": k[1], "count": len(v), "bytes": sum(v)} for k, v in groups.items()]
        return sorted(rows, key=lambda r: -r["bytes"])

    def slack(self, device) -> Optional[int]:
        """Bytes the caching allocator holds on ``device`` beyond the ledger (transients, fragmentation,
        library workspaces); None on the host."""
        dev = torch.device(device)
        if dev.type != "cuda":
            return None
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        return torch.cuda.memory_reserved(idx) - self.total_bytes(f"cuda:{idx}")

    # ------------------------------------------------------------------ red zones
    def check(self) -> List[dict]:
        """The allocations whose guard band no longer holds the pattern: name, site and how many band
        bytes changed. Empty when red zones are off or all bands are intact."""
        with self._lock:
            self._reap()
            bands = [(e.name, e.site, e.guard) for e in self._live.values() if e.guard is not None]
        bad = []
        for name, site, g in bands:
            n = int((g != PATTERN).sum())
            if n:
                first = int(torch.nonzero(g != PATTERN)[0])
                bad.append({"name": name, "site": site, "bytes_overwritten": n, "first_offset": first})
        return bad

    def refill(self) -> None:
        with self._lock:
            self._reap()
            for e in self._live.values():
                if e.guard is not None:
                    e.guard.fill_(PATTERN)


_ledger: Optional[AllocLedger] = None


def ledger() -> AllocLedger:
    """The process-wide ledger (created on first use; reads ``METRALE_REDZONE`` once)."""
    global _ledger
    if _ledger is None:
        _ledger = AllocLedger()
    return _ledger


def reset_for_tests(redzone_bytes: int = 0) -> AllocLedger:
    global _ledger
    _ledger = AllocLedger(redzone_bytes)
    return _ledger
