"""Slots for recurrent layer state (gated-delta-net / Mamba2): a conv window and an SSM matrix
per recurrent layer per live sequence, plus a snapshot area used by the prefix cache, by
speculative rollback and by sequence spill.

Slot 0 is a scratch slot for padded batch rows. Tensors are ``[num_slots, ...]`` so a batched
kernel addresses a sequence's state by slot id.
Role of the reference's SSM pool + snapshot pool (``model-engine/src/model/ssm_snapshot*.rs``,
``traits/model/ssm_state.rs``, ``scheduler/ssm_decode_ring.rs``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch


class StatePool:
    def __init__(self, layer_shapes: List[Tuple[Tuple[int, ...], Tuple[int, ...]]], num_slots: int,
                 num_snapshots: int = 0, device="cpu"):
        """layer_shapes[i] = (conv_state_shape, ssm_state_shape) of recurrent layer i."""
        self.num_slots = num_slots
        self.device = torch.device(device)
        from ..utils.alloc_ledger import ledger
        z = lambda shape, name: ledger().alloc(shape, torch.float32, device, name)
        self.conv = [z((num_slots, *c), "state pool (conv)") for c, _ in layer_shapes]
        self.ssm = [z((num_slots, *s), "state pool (ssm)") for _, s in layer_shapes]
        self._free = list(range(num_slots - 1, 0, -1))
        self.num_snapshots = num_snapshots
        self.snap_conv = [z((num_snapshots, *c), "state snapshots (conv)") for c, _ in layer_shapes]
        self.snap_ssm = [z((num_snapshots, *s), "state snapshots (ssm)") for _, s in layer_shapes]
        self._snap_free = list(range(num_snapshots - 1, -1, -1))
        self._snap_ref: Dict[int, int] = {}

    @property
    def num_layers(self) -> int:
        return len(self.conv)

    def bytes_per_slot(self) -> int:
        return sum(t[0].numel() * 4 for t in self.conv) + sum(t[0].numel() * 4 for t in self.ssm)

    # ---- live slots
    def alloc(self) -> int:
        if not self._free:
            raise RuntimeError("no free recurrent-state slot")
        s = self._free.pop()
        self.reset(s)
        return s

    def free(self, slot: int) -> None:
        if slot > 0:
            self._free.append(slot)

    def reset(self, slot: int) -> None:
        for t in self.conv + self.ssm:
            t[slot].zero_()

    @property
    def num_free(self) -> int:
        return len(self._free)

    # ---- snapshots
    # A snapshot id is a handle. Its state lives in one of three tiers: the device snapshot area
    # ("resident"), pinned host memory, or a file under `tier_dir`. When the resident area is full
    # the least recently used resident snapshot is demoted to the host tier, and the host tier
    # demotes its oldest entry to a file once `host_tier_bytes` is exceeded (when a directory is
    # configured; otherwise the host tier simply keeps growing); without tiers
    # configured a full area refuses the snapshot, as before. A hit restores from wherever the
    # snapshot is (role of the reference's resident -> tiered eviction of prefix-cache state,
    # ``crates/model-engine/src/model/ssm_snapshot_spill.rs``, ``ssm_tier/``).
    def configure_tiers(self, host_tier_bytes: int = 0, tier_dir: Optional[str] = None) -> None:
        self.host_tier_bytes, self.tier_dir = int(host_tier_bytes), tier_dir
        if tier_dir:
            import os
            os.makedirs(tier_dir, exist_ok=True)

    def _tier_init(self) -> None:
        if not hasattr(self, "_where"):
            self._where: Dict[int, tuple] = {}        # handle -> ("dev", idx) | ("host", tensors) | ("file", path)
            self._lru: List[int] = []                  # resident handles, least recently used first
            self._host_order: List[int] = []
            self._host_bytes = 0
            self._next_handle = 0
            self.host_tier_bytes = getattr(self, "host_tier_bytes", 0)
            self.tier_dir = getattr(self, "tier_dir", None)
            self.tier_stats = {"demoted_host": 0, "demoted_file": 0, "restored_host": 0, "restored_file": 0}

    def _touch(self, h: int) -> None:
        if h in self._lru:
            self._lru.remove(h)
            self._lru.append(h)

    def _demote_one(self) -> bool:
        """Move the least recently used resident snapshot down a tier; False when no tier can take it."""
        if not self._lru or (self.host_tier_bytes <= 0 and not self.tier_dir):
            return False
        h = self._lru.pop(0)
        idx = self._where[h][1]
        blob = {}
        for i in range(self.num_layers):
            blob[f"conv{i}"] = self.snap_conv[i][idx].to("cpu", copy=True)
            blob[f"ssm{i}"] = self.snap_ssm[i][idx].to("cpu", copy=True)
        self._snap_free.append(idx)
        if self.host_tier_bytes > 0:
            self._where[h] = ("host", blob)
            self._host_order.append(h)
            self._host_bytes += self.bytes_per_slot()
            self.tier_stats["demoted_host"] += 1
            while self._host_bytes > self.host_tier_bytes and self._host_order and self.tier_dir:
                old = self._host_order.pop(0)
                self._host_bytes -= self.bytes_per_slot()
                self._to_file(old, self._where[old][1])
        else:
            self._to_file(h, blob)
        return True

    def _to_file(self, h: int, blob) -> None:
        import os
        path = os.path.join(self.tier_dir, f"state_snapshot_{id(self):x}_{h}.pt")
        torch.save(blob, path)
        self._where[h] = ("file", path)
        self.tier_stats["demoted_file"] += 1

    def snapshot(self, slot: int) -> Optional[int]:
        """Copy a slot's state into the snapshot area; None when the area is full and no lower
        tier is configured."""
        self._tier_init()
        if not self._snap_free and not self._demote_one():
            return None
        idx = self._snap_free.pop()
        for i in range(self.num_layers):
            self.snap_conv[i][idx].copy_(self.conv[i][slot])
            self.snap_ssm[i][idx].copy_(self.ssm[i][slot])
        h = self._next_handle
        self._next_handle += 1
        self._where[h] = ("dev", idx)
        self._lru.append(h)
        self._snap_ref[h] = 1
        return h

    def available(self, sid: int) -> bool:
        self._tier_init()
        return sid in self._where

    def restore(self, sid: int, slot: int) -> None:
        self._tier_init()
        tier, where = self._where[sid]
        if tier == "dev":
            for i in range(self.num_layers):
                self.conv[i][slot].copy_(self.snap_conv[i][where])
                self.ssm[i][slot].copy_(self.snap_ssm[i][where])
            self._touch(sid)
            return
        blob = where if tier == "host" else torch.load(where)
        for i in range(self.num_layers):
            self.conv[i][slot].copy_(blob[f"conv{i}"])
            self.ssm[i][slot].copy_(blob[f"ssm{i}"])
        self.tier_stats["restored_host" if tier == "host" else "restored_file"] += 1

    def retain_snapshot(self, sid: int) -> None:
        self._snap_ref[sid] = self._snap_ref.get(sid, 0) + 1

    def release_snapshot(self, sid: int) -> None:
        self._tier_init()
        n = self._snap_ref.get(sid, 0) - 1
        if n > 0:
            self._snap_ref[sid] = n
            return
        self._snap_ref.pop(sid, None)
        tier, where = self._where.pop(sid, ("gone", None))
        if tier == "dev":
            self._snap_free.append(where)
            if sid in self._lru:
                self._lru.remove(sid)
        elif tier == "host":
            if sid in self._host_order:
                self._host_order.remove(sid)
                self._host_bytes -= self.bytes_per_slot()
        elif tier == "file":
            import os
            try:
                os.remove(where)
            except OSError:
                pass

    # ---- spill
    def export_slot(self, slot: int) -> Dict[str, torch.Tensor]:
        out = {}
        for i in range(self.num_layers):
            out[f"conv{i}"] = self.conv[i][slot].cpu()
            out[f"ssm{i}"] = self.ssm[i][slot].cpu()
        return out

    def import_slot(self, slot: int, data: Dict[str, torch.Tensor]) -> None:
        for i in range(self.num_layers):
            self.conv[i][slot].copy_(data[f"conv{i}"])
            self.ssm[i][slot].copy_(data[f"ssm{i}"])
