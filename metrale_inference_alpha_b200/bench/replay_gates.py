"""Three more gates over the public engine API, each split into a driver (runs requests) and decision functions
that do no I/O, so every failure class can be constructed in a test without a model.

``order_equality``   the same draw of requests is issued in two or more orders (and batched together, so batch
                     composition changes too); every sample's reply must be identical across the orders. A
                     reply that only depends on its own request passes; a reworded reply is the finding.
``conversation_replay``  a fixed multi-turn conversation is replayed N rounds against one prefix-cached engine
                     and every turn is compared with round 0. A differing turn is *collapsed* when its finish
                     reason differs or its length ratio leaves [0.5, 2.0] (early-EOS stubs, runaways: what a
                     poisoned restored state produces) and *jittered* otherwise (reworded, same shape). Collapsed,
                     unmeasured (errored) and zero-cache replays fail the run; jitter is recorded and passes. A
                     replay whose first turn restored nothing from the prefix cache proves nothing about
                     restores, so it fails too, and so does a run with fewer rounds than asked for.
``decode_floor``     single-user decode rate with every generation knob pinned (prompt, temperature 0, seed 0,
                     token count), median over several runs, judged against a floor.

Reference: ``crates/bench/src/benchmarks/kat_equality/{compare,driver}.rs``, ``ssm_poison/{compare,score,driver}.rs``,
``decode_floor/mod.rs``.
"""
from __future__ import annotations

import statistics
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..sampling.params import SamplingParams
from .gate import GateRecord, kernel_closure_hash

COLLAPSE_RATIO_FLOOR, COLLAPSE_RATIO_CEIL = 0.5, 2.0


# ----------------------------------------------------------------------------- order equality
def compare_orders(replies: Sequence[Dict[str, Sequence[int]]]) -> dict:
    """``replies[o][sample_id]`` = the reply of that sample in order o. Passes only with at least two orders, at
    least one sample, not every reference reply empty, and every sample equal in every order."""
    if len(replies) < 2:
        return {"pass": False, "why": "fewer than two orders", "unequal": []}
    ref = replies[0]
    if not ref:
        return {"pass": False, "why": "no samples", "unequal": []}
    if all(len(v) == 0 for v in ref.values()):
        return {"pass": False, "why": "every reference reply is empty", "unequal": []}
    unequal = []
    for sid, want in ref.items():
        for o, rep in enumerate(replies[1:], 1):
            got = rep.get(sid)
            if got is None or list(got) != list(want):
                k = len(want) if got is None else next((j for j, (a, b) in enumerate(zip(got, want)) if a != b), min(len(got), len(want)))
                unequal.append({"sample": sid, "order": o, "first_difference": k, "missing": got is None})
                break
    return {"pass": not unequal, "why": "" if not unequal else f"{len(unequal)} of {len(ref)} samples differ between orders",
            "unequal": unequal}


def order_equality(engine, prompts: Sequence[Sequence[int]], orders: int = 3, max_tokens: int = 16, seed: int = 0,
                   device: str = "") -> GateRecord:
    import random
    ids = [f"s{i}" for i in range(len(prompts))]
    rng = random.Random(seed)
    replies = []
    for o in range(orders):
        perm = list(range(len(prompts)))
        if o:
            rng.shuffle(perm)
        sps = [SamplingParams(max_tokens=max_tokens, temperature=0.0, ignore_eos=True) for _ in perm]
        outs = engine.generate([list(prompts[i]) for i in perm], sps)
        replies.append({ids[i]: list(out.output_ids) for i, out in zip(perm, outs)})
    res = compare_orders(replies)
    return GateRecord("order-equality", "every sample's reply identical across request orders", 1.0 if res["pass"] else 0.0,
                      "pass", config={"orders": orders, "samples": len(prompts), "max_tokens": max_tokens, **res,
                                      "model": engine.cfg.name}, closure=kernel_closure_hash(), device=device)


# ----------------------------------------------------------------------------- conversation replay
@dataclass
class Turn:
    tokens: List[int]
    finish_reason: Optional[str]
    cached_tokens: int = 0
    error: str = ""


def compare_turn(ref: Turn, got: Turn) -> str:
    if got.error:
        return "unmeasured"
    if got.tokens == ref.tokens and got.finish_reason == ref.finish_reason:
        return "invariant"
    ratio = len(got.tokens) / max(1, len(ref.tokens))
    if got.finish_reason != ref.finish_reason or not (COLLAPSE_RATIO_FLOOR <= ratio <= COLLAPSE_RATIO_CEIL):
        return "collapsed"
    return "jittered"


def compare_round(ref: Sequence[Turn], got: Sequence[Turn]) -> str:
    """Collapsed if any turn collapsed, else unmeasured if any turn was (or the round is short), else jittered if
    any turn jittered, else invariant."""
    verdicts = [compare_turn(r, g) for r, g in zip(ref, got)]
    if len(got) < len(ref):
        verdicts.append("unmeasured")
    for v in ("collapsed", "unmeasured", "jittered"):
        if v in verdicts:
            return v
    return "invariant"


@dataclass
class ReplayScore:
    rounds_wanted: int
    verdicts: List[str] = field(default_factory=list)
    zero_cache_rounds: List[int] = field(default_factory=list)
    reference_ok: bool = True

    def decide(self) -> dict:
        why = []
        if not self.reference_ok:
            why.append("the reference round does not meet the script's anchors")
        if len(self.verdicts) < self.rounds_wanted:
            why.append(f"short run: {len(self.verdicts)} of {self.rounds_wanted} replays")
        for v in ("collapsed", "unmeasured"):
            n = self.verdicts.count(v)
            if n:
                why.append(f"{n} {v} replay(s)")
        if self.zero_cache_rounds:
            why.append(f"replays {self.zero_cache_rounds} restored nothing from the prefix cache")
        return {"pass": not why, "why": "; ".join(why), "jittered": self.verdicts.count("jittered"),
                "invariant": self.verdicts.count("invariant")}


def conversation_replay(engine, script: Sequence[Sequence[int]], rounds: int = 12, max_tokens: int = 12,
                        noise: Optional[Callable[[int], None]] = None, min_reference_tokens: int = 1,
                        device: str = "") -> GateRecord:
    """``script``: the user turns as token lists. A round feeds turn 1, appends the reply, feeds turn 2 behind it, and
    so on (the growing conversation is what the prefix cache and the recurrent-state snapshots serve). ``noise(r)``
    runs between rounds (other traffic that recycles blocks and state slots). The anchor asked of the reference
    round is that every turn produced at least ``min_reference_tokens`` tokens and finished by length or stop."""
    def one_round() -> List[Turn]:
        turns, history = [], []
        for user in script:
            history = history + list(user)
            try:
                out = engine.generate([history], SamplingParams(max_tokens=max_tokens, temperature=0.0))[0]
                turns.append(Turn(list(out.output_ids), out.finish_reason, out.cached_tokens))
                history = history + list(out.output_ids)
            except Exception as e:                                      # a failed round is scored, the run goes on
                turns.append(Turn([], None, 0, error=f"{type(e).__name__}: {e}"))
                break
        return turns
    ref = one_round()
    score = ReplayScore(rounds)
    score.reference_ok = len(ref) == len(script) and all(not t.error and len(t.tokens) >= min_reference_tokens for t in ref)
    for r in range(1, rounds + 1):
        if noise is not None:
            noise(r)
        got = one_round()
        score.verdicts.append(compare_round(ref, got))
        if got and not got[0].error and got[0].cached_tokens == 0:
            score.zero_cache_rounds.append(r)
    res = score.decide()
    return GateRecord("conversation-replay", f"{rounds} replays of a {len(script)}-turn conversation: none collapsed",
                      1.0 if res["pass"] else 0.0, "pass",
                      config={"rounds": rounds, "turns": len(script), "verdicts": score.verdicts, **res, "model": engine.cfg.name},
                      closure=kernel_closure_hash(), device=device)


# ----------------------------------------------------------------------------- decode floor
def judge_floor(rates: Sequence[float], floor: float, min_runs: int = 3) -> dict:
    if len(rates) < min_runs:
        return {"pass": False, "why": f"{len(rates)} of {min_runs} runs", "median": 0.0}
    med = statistics.median(rates)
    return {"pass": med >= floor, "why": "" if med >= floor else f"median {med:.1f} tok/s is under the floor {floor:.1f}", "median": med}


def decode_floor(engine, prompt: Sequence[int], floor_tok_s: float, runs: int = 5, max_tokens: int = 64,
                 device: str = "") -> GateRecord:
    rates = []
    for _ in range(runs):
        sp = SamplingParams(max_tokens=max_tokens, temperature=0.0, seed=0, ignore_eos=True)
        t0 = time.perf_counter()
        out = engine.generate([list(prompt)], sp)[0]
        wall = time.perf_counter() - t0
        # the engine's own decode time when it reports one (prefill excluded), else wall clock of the request
        dec_s = out.decode_ms / 1e3 if out.decode_ms else wall
        rates.append((len(out.output_ids) - 1) / dec_s if dec_s > 0 and len(out.output_ids) > 1 else 0.0)
    res = judge_floor(rates, floor_tok_s, min_runs=min(3, runs))
    return GateRecord("decode-floor", "single-user decode tok/s, median of pinned runs", res["median"], "tokens/s",
                      config={"runs": runs, "max_tokens": max_tokens, "floor": floor_tok_s, "rates": [round(r, 2) for r in rates],
                              "pass": res["pass"], "why": res["why"], "model": engine.cfg.name},
                      closure=kernel_closure_hash(), device=device)
