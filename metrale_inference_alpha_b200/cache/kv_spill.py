"""Swap preempted sequences out instead of recomputing them: the sequence's KV blocks (every
layer) and its recurrent-state slot are gathered into pinned host memory (tier 1) and, past a
host budget, written to a swap file (tier 2); on re-admission fresh blocks are allocated and the
bytes scattered back, so decode continues where it stopped without re-running the prefill.

The scheduler core calls ``save(seq, core)`` / ``restore(seq, core)`` (``SchedulerConfig.
preempt_mode = "swap"``). Role of the reference's ``KvSpillManager`` swap files
(``crates/cache/src/kv_spill.rs``) and the ``SpillIo`` effect of ``crates/scheduler``.
"""
from __future__ import annotations

import os
import tempfile
from typing import Dict, Optional

import torch


class KvSpillManager:
    def __init__(self, kv, state_pool=None, host_budget_bytes: int = 8 << 30, swap_dir: Optional[str] = None):
        self.kv, self.pool = kv, state_pool
        self.host_budget = host_budget_bytes
        self.swap_dir = swap_dir or os.path.join(tempfile.gettempdir(), f"metrale_kv_swap_{os.getpid()}")
        self._host: Dict[int, dict] = {}
        self._host_bytes = 0
        self.stats = {"saved": 0, "restored": 0, "to_disk": 0, "bytes_out": 0, "bytes_in": 0, "refused": 0}

    @staticmethod
    def _nbytes(blob: dict) -> int:
        return sum(t.numel() * t.element_size() for t in blob.values() if isinstance(t, torch.Tensor))

    # ------------------------------------------------------------------ scheduler hooks
    def save(self, seq, core) -> bool:
        """Copy the sequence's cached tokens out and release its blocks. False = could not (the
        scheduler then falls back to recompute)."""
        nblk = (seq.num_computed + core.cfg.block_size - 1) // core.cfg.block_size
        if nblk == 0 or nblk > len(seq.blocks):
            self.stats["refused"] += 1
            return False
        try:
            blob = {k: v.to("cpu", non_blocking=False) for k, v in self.kv.gather_blocks(seq.blocks[:nblk]).items()}
            if self.pool is not None and seq.state_slot:
                for k, v in self.pool.export_slot(seq.state_slot).items():
                    blob["state." + k] = v.to("cpu")
        except Exception:
            self.stats["refused"] += 1
            return False
        n = self._nbytes(blob)
        if self._host_bytes + n > self.host_budget:
            os.makedirs(self.swap_dir, exist_ok=True)
            path = os.path.join(self.swap_dir, f"seq{seq.seq_id}.pt")
            torch.save(blob, path)
            seq.swap_file = path
            self.stats["to_disk"] += 1
        else:
            self._host[seq.seq_id] = blob
            self._host_bytes += n
        seq.swapped_blocks = nblk
        core.alloc.free(seq.blocks)
        seq.blocks = []
        if self.pool is not None and seq.state_slot:
            self.pool.free(seq.state_slot)
            seq.state_slot = 0
        self.stats["saved"] += 1
        self.stats["bytes_out"] += n
        return True

    def restore(self, seq, core) -> None:
        blob = self._host.pop(seq.seq_id, None)
        if blob is not None:
            self._host_bytes -= self._nbytes(blob)
        else:
            blob = torch.load(seq.swap_file)
            os.remove(seq.swap_file)
            seq.swap_file = None
        nblk = seq.swapped_blocks
        seq.blocks = core._alloc_blocks(nblk)
        kvb = {k: v for k, v in blob.items() if not k.startswith("state.")}
        self.kv.scatter_blocks(seq.blocks, {k: v.to(self.kv.device) for k, v in kvb.items()})
        if self.pool is not None:
            st = {k[6:]: v for k, v in blob.items() if k.startswith("state.")}
            if st:
                seq.state_slot = self.pool.alloc()
                self.pool.import_slot(seq.state_slot, {k: v.to(self.pool.device) for k, v in st.items()})
        self.stats["restored"] += 1
        self.stats["bytes_in"] += self._nbytes(blob)

    def drop(self, seq) -> None:
        """Forget a swapped-out sequence (abort / timeout while swapped)."""
        blob = self._host.pop(seq.seq_id, None)
        if blob is not None:
            self._host_bytes -= self._nbytes(blob)
        if getattr(seq, "swap_file", None):
            try:
                os.remove(seq.swap_file)
            except OSError:
                pass
            seq.swap_file = None
