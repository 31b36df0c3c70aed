"""Executors that need no model: a scripted one (answers every sampled row from a script or a
function, can inject KV exhaustion and fatal faults) and a tracing wrapper that records every
plan. They let the scheduler core be tested on a machine without a GPU.
Role of the reference's ``ScriptedDeviceIo`` / ``TracingDeviceIo`` (``crates/scheduler/src/scripted.rs``).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

from .types import FatalDeviceError, KvExhausted, StepPlan, StepResult


class ScriptedExecutor:
    def __init__(self, token_fn: Optional[Callable[[int, int], int]] = None, vocab: int = 1000):
        """token_fn(seq_id, position) -> token id produced after the token at `position`."""
        self.token_fn = token_fn or (lambda sid, pos: (sid * 7919 + pos * 31) % vocab)
        self.faults: Dict[int, str] = {}       # step index -> "kv" | "fatal"
        self.steps = 0
        self.draft_fn: Optional[Callable[[int, int, int], List[int]]] = None

    def inject(self, step: int, kind: str) -> None:
        self.faults[step] = kind

    def execute(self, plan: StepPlan) -> StepResult:
        fault = self.faults.pop(self.steps, None)
        self.steps += 1
        if fault == "kv":
            raise KvExhausted("scripted")
        if fault == "fatal":
            raise FatalDeviceError("scripted")
        toks = []
        for it in plan.items:
            if not it.sample:
                toks.append([])
                continue
            sid = it.seq.seq_id
            base = it.start_pos
            rows = range(len(it.tokens) - 1 - it.verify, len(it.tokens))
            toks.append([self.token_fn(sid, base + r) for r in rows])
        return StepResult(toks)

    def propose(self, plan: StepPlan, result: StepResult, k: int) -> List[List[int]]:
        if self.draft_fn is None:
            return [[] for _ in plan.items]
        return [self.draft_fn(it.seq.seq_id, len(it.seq.tokens), k) for it in plan.items]


class TracingExecutor:
    def __init__(self, inner):
        self.inner = inner
        self.trace: List[dict] = []

    def execute(self, plan: StepPlan) -> StepResult:
        self.trace.append({"kind": plan.kind, "tokens": plan.num_tokens,
                           "seqs": [(i.seq.seq_id, i.start_pos, len(i.tokens), i.verify) for i in plan.items]})
        return self.inner.execute(plan)

    def __getattr__(self, name):
        return getattr(self.inner, name)
