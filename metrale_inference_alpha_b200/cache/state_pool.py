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
        self.conv = [torch.zeros((num_slots, *c), dtype=torch.float32, device=device) for c, _ in layer_shapes]
        self.ssm = [torch.zeros((num_slots, *s), dtype=torch.float32, device=device) for _, s in layer_shapes]
        self._free = list(range(num_slots - 1, 0, -1))
        self.num_snapshots = num_snapshots
        self.snap_conv = [torch.zeros((num_snapshots, *c), dtype=torch.float32, device=device) for c, _ in layer_shapes]
        self.snap_ssm = [torch.zeros((num_snapshots, *s), dtype=torch.float32, device=device) for _, s in layer_shapes]
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
    def snapshot(self, slot: int) -> Optional[int]:
        """Copy a slot's state into the snapshot area; None when the area is full."""
        if not self._snap_free:
            return None
        sid = self._snap_free.pop()
        for i in range(self.num_layers):
            self.snap_conv[i][sid].copy_(self.conv[i][slot])
            self.snap_ssm[i][sid].copy_(self.ssm[i][slot])
        self._snap_ref[sid] = 1
        return sid

    def restore(self, sid: int, slot: int) -> None:
        for i in range(self.num_layers):
            self.conv[i][slot].copy_(self.snap_conv[i][sid])
            self.ssm[i][slot].copy_(self.snap_ssm[i][sid])

    def release_snapshot(self, sid: int) -> None:
        n = self._snap_ref.get(sid, 0) - 1
        if n <= 0:
            self._snap_ref.pop(sid, None)
            self._snap_free.append(sid)
        else:
            self._snap_ref[sid] = n

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
