"""Multi-rank control plane: rank 0 owns HTTP; before every engine tick it publishes the
operations that arrived since the last tick (add / abort / shutdown) and every rank applies
the same list in the same order, so all ranks' schedulers make identical decisions and issue
identical collectives (SPMD). A heartbeat on the rendezvous store lets a rank learn that a
peer left *before* its next launch. Role of the reference's rank-0 broadcast of step plans and
its worker watchdog (``crates/server/src/main_modules/tp_worker.rs``,
``crates/comm/src/collective_wait.rs``).

The payload travels over a CPU (gloo) group: control traffic never waits behind GPU work and a
dead peer ends the broadcast with a timeout instead of a stuck kernel.
"""
from __future__ import annotations

import pickle
import threading
import time
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Any, List, Optional, Tuple

import torch
import torch.distributed as dist

Op = Tuple[str, Any, Any, Any]          # (kind, request_id, prompt_ids, params)


class PeerLost(RuntimeError):
    pass


@dataclass
class ControlPlane:
    rank: int
    size: int
    group: Optional[Any] = None           # a gloo group; None when size == 1
    store: Optional[Any] = None           # c10d store for heartbeats
    heartbeat_s: float = 1.0
    dead_after_s: float = 5.0
    _hb_thread: Optional[threading.Thread] = field(default=None, repr=False)
    _stop: threading.Event = field(default_factory=threading.Event, repr=False)
    ticks: int = 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, timeout_s: float = 30.0, heartbeat: bool = True) -> "ControlPlane":
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return cls(0, 1)
        group = dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_s))
        store = None
        try:
            store = dist.distributed_c10d._get_default_store()
        except Exception:
            pass
        cp = cls(dist.get_rank(), dist.get_world_size(), group, store)
        if heartbeat and store is not None:
            cp.start_heartbeat()
        return cp

    # ------------------------------------------------------------------ per-tick exchange
    def exchange(self, ops: Optional[List[Op]]) -> List[Op]:
        """Rank 0 passes the operations it collected; every rank returns the same list."""
        self.ticks += 1
        if self.size == 1:
            return ops or []
        if self.rank == 0:
            blob = pickle.dumps(ops or [])
            n = torch.tensor([len(blob)], dtype=torch.int64)
        else:
            n = torch.zeros(1, dtype=torch.int64)
        try:
            dist.broadcast(n, src=0, group=self.group)
            if int(n) == 0:
                return []
            buf = torch.frombuffer(bytearray(blob), dtype=torch.uint8) if self.rank == 0 else \
                torch.empty(int(n), dtype=torch.uint8)
            dist.broadcast(buf, src=0, group=self.group)
        except RuntimeError as e:
            raise PeerLost(f"control broadcast failed on rank {self.rank}: {e}") from e
        if self.rank == 0:
            return ops or []
        return pickle.loads(buf.numpy().tobytes())

    def agree(self, ok: bool) -> bool:
        """All ranks report health; returns True only when every rank is healthy."""
        if self.size == 1:
            return ok
        t = torch.tensor([1 if ok else 0], dtype=torch.int32)
        try:
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        except RuntimeError as e:
            raise PeerLost(f"health agreement failed on rank {self.rank}: {e}") from e
        return bool(int(t))

    # ------------------------------------------------------------------ heartbeats
    def start_heartbeat(self) -> None:
        def beat():
            while not self._stop.is_set():
                try:
                    self.store.set(f"hb/{self.rank}", str(time.time()))
                except Exception:
                    return
                self._stop.wait(self.heartbeat_s)
        self._hb_thread = threading.Thread(target=beat, name="heartbeat", daemon=True)
        self._hb_thread.start()

    def lost_peers(self, now: Optional[float] = None) -> List[int]:
        """Ranks whose heartbeat is older than ``dead_after_s`` (or that announced leaving)."""
        if self.store is None or self.size == 1:
            return []
        now = time.time() if now is None else now
        lost = []
        for r in range(self.size):
            if r == self.rank:
                continue
            try:
                if not self.store.check([f"hb/{r}"]):
                    continue                      # never started: not counted as lost
                v = self.store.get(f"hb/{r}").decode()
            except Exception:
                lost.append(r)
                continue
            if v == "left" or now - float(v) > self.dead_after_s:
                lost.append(r)
        return lost

    def check_peers(self) -> None:
        lost = self.lost_peers()
        if lost:
            raise PeerLost(f"rank {self.rank}: peers {lost} stopped sending heartbeats")

    def leave(self) -> None:
        """Announce an orderly exit (between steps, nothing in flight)."""
        self._stop.set()
        if self.store is not None:
            try:
                self.store.set(f"hb/{self.rank}", "left")
            except Exception:
                pass


def follower_loop(engine, cp: ControlPlane, max_ticks: Optional[int] = None) -> str:
    """Ranks > 0: apply rank 0's operations and step in lockstep until told to stop.
    Returns the reason the loop ended ('shutdown', 'peer_lost: ...', 'fault: ...')."""
    n = 0
    while max_ticks is None or n < max_ticks:
        n += 1
        try:
            cp.check_peers()
            ops = cp.exchange(None)
        except PeerLost as e:
            engine.fault.set(str(e))
            return f"peer_lost: {e}"
        for kind, rid, ids, params in ops:
            if kind == "add":
                try:
                    engine.add_request(ids, params, request_id=rid)
                except Exception:
                    pass                              # rank 0 rejected it the same way
            elif kind == "abort":
                engine.abort(rid)
            elif kind == "shutdown":
                cp.leave()
                return "shutdown"
        if engine.has_work():
            try:
                engine.step()
            except Exception as e:
                engine.fault.set(f"{type(e).__name__}: {e}")
                return f"fault: {e}"
    return "max_ticks"
