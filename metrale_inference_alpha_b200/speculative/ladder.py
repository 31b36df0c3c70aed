"""Draft-width policies.

* ``KLadder``: drafts per sequence as a function of batch width, default ``4:3,8:3,16:1,32:1``
  (``crates/model-layers/src/speculative/ladder.rs:1-26``).
* ``spec_capacity``: tiered verify slots: slots 0..8 hold 3 drafts, the rest hold 1
  (``crates/speculative/src/spec_capacity.rs:11-20``).
* ``AdaptiveRung``: 1 <-> 2 drafts for widths 9..16 from an EWMA of the expected token ratio
  with enter / leave hysteresis (``crates/speculative/src/adaptive_rung.rs:1-28``).
* ``DflashRung``: block-drafter width: `multi` at C >= 2; at C = 1 wide / narrow by the
  popcount of first-draft accepts over a 64-step window (``crates/speculative/src/dflash_rung.rs:1-47``).
* ``dcut_plan``: prune low-confidence draft positions by the prefix sum of top-1 log-probs,
  keeping a ratio in {0.25, 0.5, 0.75, 1}; the first draft is never pruned; verify rows are
  capped (``crates/server/src/scheduler/mtp_dcut.rs:1-37``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Sequence

VERIFY_ROW_CAP = 256


class KLadder:
    DEFAULT = "4:3,8:3,16:1,32:1"

    def __init__(self, spec: str = None, max_k: int = 4):
        spec = spec or os.environ.get("METRALE_MTP_K_LADDER", self.DEFAULT)
        self.rungs = sorted((int(a), int(b)) for a, b in (p.split(":") for p in spec.split(",") if p))
        self.max_k = max_k

    def drafts_for(self, batch_width: int) -> int:
        for width, k in self.rungs:
            if batch_width <= width:
                return min(k, self.max_k)
        return 0            # wider than the ladder: no speculation


def spec_capacity(slot: int, tier_slots: int = 8, wide: int = 3, narrow: int = 1) -> int:
    return wide if slot < tier_slots else narrow


def step_drafts(slots: Sequence[int], ladder: KLadder) -> int:
    if not slots:
        return 0
    return min(ladder.drafts_for(len(slots)), min(spec_capacity(s) for s in slots))


class AdaptiveRung:
    def __init__(self, enter: float = 1.35, leave: float = 1.2, alpha: float = 0.1):
        self.enter, self.leave, self.alpha = enter, leave, alpha
        self.k = 1
        self.p1 = 0.5
        self.p2 = 0.5

    def observe(self, first_accepted: bool, second_accepted: bool = False) -> None:
        self.p1 += self.alpha * ((1.0 if first_accepted else 0.0) - self.p1)
        if first_accepted:
            self.p2 += self.alpha * ((1.0 if second_accepted else 0.0) - self.p2)

    def token_ratio(self) -> float:
        """Expected tokens per step with two drafts relative to one."""
        return (1 + self.p1 + self.p1 * self.p2) / (1 + self.p1)

    def drafts(self, width: int) -> int:
        if not 9 <= width <= 16:
            return self.k if width < 9 else 1
        r = self.token_ratio() * (1 + self.p1)
        if self.k == 1 and r > self.enter + self.p1:
            self.k = 2
        elif self.k == 2 and r < self.leave + self.p1:
            self.k = 1
        return self.k


class DflashRung:
    def __init__(self, multi: int = 4, wide: int = 8, narrow: int = 5, window: int = 64, dwell: int = 16):
        self.multi, self.wide, self.narrow, self.window, self.dwell = multi, wide, narrow, window, dwell
        self.bits: List[int] = []
        self.current = narrow
        self._since = 0

    def observe(self, first_draft_accepted: bool) -> None:
        self.bits.append(1 if first_draft_accepted else 0)
        if len(self.bits) > self.window:
            self.bits.pop(0)
        self._since += 1

    def gamma(self, concurrency: int) -> int:
        if concurrency >= 2:
            return self.multi
        if self._since >= self.dwell and len(self.bits) >= self.window // 2:
            frac = sum(self.bits) / len(self.bits)
            want = self.wide if frac > 0.6 else self.narrow
            if want != self.current:
                self.current, self._since = want, 0
        return self.current


def dcut_plan(logprobs: Sequence[Sequence[float]], ratio: float = 1.0, row_cap: int = VERIFY_ROW_CAP
              ) -> List[int]:
    """Per sequence, how many of its drafts to verify. `logprobs[s][j]` is the drafter's
    top-1 log-prob of draft j. Survival score = prefix sum; the lowest-scoring prunable
    positions are cut first, suffix-closed (cutting j cuts everything after it)."""
    assert ratio in (0.25, 0.5, 0.75, 1.0)
    keep = [len(lp) for lp in logprobs]
    prunable = []
    for s, lp in enumerate(logprobs):
        acc = 0.0
        for j, v in enumerate(lp):
            acc += v
            if j >= 1:
                prunable.append((acc, s, j))
    total = sum(keep) + len(keep)                   # + one bonus row per sequence
    target_cut = int(round(len(prunable) * (1.0 - ratio)))
    prunable.sort()
    cut = 0
    for score, s, j in prunable:
        over_cap = total > row_cap
        if cut >= target_cut and not over_cap:
            break
        if j < keep[s]:
            removed = keep[s] - j
            keep[s] = j
            total -= removed
            cut += removed
    return keep
