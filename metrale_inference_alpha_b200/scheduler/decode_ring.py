"""Decode-time ring of recurrent-state snapshots of one sequence.

Rolling a generation back to an earlier token (a loop detector that rewinds to the last sentence
boundary, a tool-call parser that rejects a malformed tail) only needs the KV cache to be
truncated for attention layers, but a recurrent layer's state cannot be rewound: it has to be
restored from a snapshot taken when exactly that many tokens had been generated. The ring keeps
the newest `capacity` such snapshots; recording into a full ring evicts the oldest. It holds
snapshot handles of the state pool, nothing on the device itself.

Role of the reference's ``crates/server/src/scheduler/ssm_decode_ring.rs`` (bounded entries,
``token_position`` = generated tokens when the snapshot was taken, rollback needs an exact match).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional


@dataclass
class RingEntry:
    token_position: int      # number of generated tokens when the snapshot was taken
    snapshot: int            # state-pool snapshot handle


class StateDecodeRing:
    def __init__(self, capacity: int):
        self.capacity = max(0, int(capacity))
        self.entries: List[RingEntry] = []       # oldest first

    def record(self, token_position: int, snapshot: int) -> Optional[int]:
        """Add an entry; returns the handle of the evicted (or refused) snapshot to release, if any."""
        if self.capacity == 0:
            return snapshot
        drop = None
        # a re-generated position (after a rollback) replaces the stale entry
        for e in self.entries:
            if e.token_position == token_position:
                drop, e.snapshot = e.snapshot, snapshot
                return drop
        if len(self.entries) == self.capacity:
            drop = self.entries.pop(0).snapshot
        self.entries.append(RingEntry(token_position, snapshot))
        return drop

    def find(self, keep_len: int) -> Optional[RingEntry]:
        for e in self.entries:
            if e.token_position == keep_len:
                return e
        return None

    def positions(self) -> List[int]:
        return [e.token_position for e in self.entries]

    def last_at_or_before(self, keep_len: int) -> Optional[RingEntry]:
        best = None
        for e in self.entries:
            if e.token_position <= keep_len and (best is None or e.token_position > best.token_position):
                best = e
        return best

    def truncate_after(self, keep_len: int) -> List[int]:
        """Forget entries newer than `keep_len`; returns their snapshot handles."""
        gone = [e.snapshot for e in self.entries if e.token_position > keep_len]
        self.entries = [e for e in self.entries if e.token_position <= keep_len]
        return gone

    def clear(self) -> List[int]:
        gone = [e.snapshot for e in self.entries]
        self.entries = []
        return gone
