"""Change ledger: an append-only JSON-lines journey per pull request. Every line is one event
(``state`` change, ``gate`` verdict, ``category`` label, ``measurement`` with named metrics) stamped
with the PR number, head commit, CI run and attempt. Reading gives the journey; ``deduplicated``
drops replays of the same (commit, run, attempt, payload); ``materialize`` turns it into a small
graph (commit nodes -observed-> event nodes, events of one PR chained by -precedes->) that the
queries below walk: the latest verdict of every gate at a commit, gates invalidated by a later
event, and whether the PR may merge.

Role of the reference's ``crates/governance`` (``event.rs``, ``ledger.rs``); its gate records are
``bench/gate.py``.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

VERDICTS = ("pass", "fail", "missing")
KINDS = ("state", "gate", "category", "measurement")


@dataclass
class Event:
    pr: int
    head_sha: str
    kind: str
    at: int = 0
    run_id: str = ""
    attempt: int = 0
    payload: Dict[str, object] = field(default_factory=dict)

    def __post_init__(self):
        if self.kind not in KINDS:
            raise ValueError(f"unknown event kind {self.kind!r}")
        if self.kind == "gate" and self.payload.get("verdict") not in VERDICTS:
            raise ValueError("gate event needs verdict pass | fail | missing")
        if not self.at:
            self.at = int(time.time())

    # ---- constructors
    @classmethod
    def state(cls, pr, sha, to, **kw):
        return cls(pr, sha, "state", payload={"to": to}, **kw)

    @classmethod
    def gate(cls, pr, sha, gate_id, verdict, invalidated_by: Iterable[str] = (), detail: Optional[str] = None, **kw):
        p: Dict[str, object] = {"id": gate_id, "verdict": verdict}
        if invalidated_by:
            p["invalidated_by"] = list(invalidated_by)
        if detail is not None:
            p["detail"] = detail
        return cls(pr, sha, "gate", payload=p, **kw)

    @classmethod
    def category(cls, pr, sha, value, status, **kw):
        return cls(pr, sha, "category", payload={"value": value, "status": status}, **kw)

    @classmethod
    def measurement(cls, pr, sha, benchmark, metrics: Dict[str, float], **kw):
        return cls(pr, sha, "measurement", payload={"benchmark": benchmark, "metrics": dict(sorted(metrics.items()))}, **kw)

    # ---- wire form: the payload is flattened beside the envelope, tagged by "kind"
    def to_json(self) -> str:
        d = {"pr": self.pr, "head_sha": self.head_sha, "run_id": self.run_id, "attempt": self.attempt, "at": self.at,
             "kind": self.kind, **self.payload}
        return json.dumps(d, sort_keys=True, separators=(",", ":"))

    @classmethod
    def from_json(cls, line: str) -> "Event":
        d = json.loads(line)
        env = {k: d.pop(k) for k in ("pr", "head_sha", "kind")}
        opt = {k: d.pop(k) for k in ("run_id", "attempt", "at") if k in d}
        return cls(env["pr"], env["head_sha"], env["kind"], payload=d, **opt)

    def identity(self) -> str:
        return "|".join([self.head_sha, self.run_id, str(self.attempt), self.kind,
                         json.dumps(self.payload, sort_keys=True, separators=(",", ":"))])


@dataclass
class Journey:
    events: List[Event] = field(default_factory=list)

    def deduplicated(self) -> "Journey":
        seen, out = set(), []
        for e in self.events:
            k = e.identity()
            if k not in seen:
                seen.add(k)
                out.append(e)
        return Journey(out)

    def gate_history(self, gate_id: str) -> List[Event]:
        return [e for e in self.events if e.kind == "gate" and e.payload.get("id") == gate_id]

    def latest_gates(self, head_sha: Optional[str] = None) -> Dict[str, Event]:
        """Latest event per gate (optionally only those observed at `head_sha`)."""
        out: Dict[str, Event] = {}
        for e in self.events:
            if e.kind == "gate" and (head_sha is None or e.head_sha == head_sha):
                out[str(e.payload["id"])] = e
        return out

    def head(self) -> Optional[str]:
        return self.events[-1].head_sha if self.events else None

    def mergeable(self, required: Iterable[str]) -> Tuple[bool, List[str]]:
        """Every required gate has passed at the newest commit and nothing later invalidated it."""
        sha = self.head()
        gates = self.latest_gates(sha)
        later_ids = {}
        for i, e in enumerate(self.events):
            if e.kind == "gate":
                later_ids[str(e.payload["id"])] = i
        blockers = []
        for g in required:
            e = gates.get(g)
            if e is None:
                blockers.append(f"{g}: missing at {sha}")
                continue
            if e.payload["verdict"] != "pass":
                blockers.append(f"{g}: {e.payload['verdict']}")
                continue
            mine = self.events.index(e)
            for other in e.payload.get("invalidated_by", []):
                if later_ids.get(other, -1) > mine:
                    blockers.append(f"{g}: invalidated by a later {other}")
        return (not blockers), blockers


def path_for(root, pr: int) -> Path:
    return Path(root) / "journeys" / f"pr-{pr}.jsonl"


def append(path, event: Event) -> None:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    line = (event.to_json() + "\n").encode()
    fd = os.open(p, os.O_WRONLY | os.O_CREAT | os.O_APPEND, 0o644)      # one write: whole lines only
    try:
        os.write(fd, line)
    finally:
        os.close(fd)


def read_all(path) -> Journey:
    events = []
    with open(path, "r", encoding="utf-8") as f:
        for n, line in enumerate(f, 1):
            if not line.strip():
                continue
            try:
                events.append(Event.from_json(line))
            except (ValueError, KeyError) as e:
                raise ValueError(f"{path} line {n}: {e}") from None
    return Journey(events)


@dataclass
class Graph:
    nodes: List[dict] = field(default_factory=list)                       # {"label", ...fields}
    edges: List[Tuple[int, int, str]] = field(default_factory=list)       # (from, to, relation)

    def out(self, node: int, relation: str) -> List[int]:
        return [b for a, b, r in self.edges if a == node and r == relation]


def materialize(journey: Journey) -> Graph:
    g = Graph()
    commits = sorted({e.head_sha for e in journey.events})
    index = {sha: i for i, sha in enumerate(commits)}
    for sha in commits:
        g.nodes.append({"label": "commit", "sha": sha})
    base = len(commits)
    last_of_pr: Dict[int, int] = {}
    for i, e in enumerate(journey.events):
        g.nodes.append({"label": e.kind, "at": e.at, "pr": e.pr, **e.payload})
        g.edges.append((index[e.head_sha], base + i, "observed"))
        if e.pr in last_of_pr:
            g.edges.append((last_of_pr[e.pr], base + i, "precedes"))
        last_of_pr[e.pr] = base + i
    return g
