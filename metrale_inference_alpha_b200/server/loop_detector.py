"""Cross-turn repetition detection for agent loops: when the recent assistant turns of a
conversation keep saying (or calling) nearly the same thing, the next turn is nudged away from
another tool call.

Each assistant message becomes a signature of three channels: hashed 4-token shingles of its text,
of its tool-call names + arguments, and of both together; a channel with fewer than 8 tokens is
empty. Newest first, adjacent signatures are compared per channel by Jaccard similarity; a *run*
is the leading streak of pairs at or above 0.50.

* hint: a run of 2 turns whose pair reaches 0.65, or of 3 turns -> a soft negative logit bias on
  the tool-call opener, growing with the run;
* suppress: a run of 4 or more turns, or of 3 with a pair at 0.65 -> the opener is masked for
  this turn, unless every repeated call failed (the model is retrying an error), the tool results
  still change from round to round (the loop is making progress), or
  ``METRALE_LOOP_NO_SUPPRESS=1``; then only the soft bias applies.

Role of the reference's ``crates/server/src/loop_detector.rs`` and ``api/chat/loop_detect.rs``.
"""
from __future__ import annotations

import json
import os
import re
import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Set

SHINGLE_ORDER = 4
MAX_SIGNATURES = 6
MIN_CHANNEL_TOKENS = 8
HIGH_SIMILARITY = 0.65
MODERATE_SIMILARITY = 0.50
CHANNELS = ("text", "calls", "both")
_TOKEN = re.compile(r"\w+|[^\w\s]")


def _shingles(tokens: List[str]) -> Set[int]:
    if len(tokens) < MIN_CHANNEL_TOKENS:
        return set()
    return {zlib.crc32(" ".join(tokens[i:i + SHINGLE_ORDER]).encode()) for i in range(len(tokens) - SHINGLE_ORDER + 1)}


def signature(message: dict) -> Dict[str, Set[int]]:
    c = message.get("content")
    if isinstance(c, list):
        c = " ".join(p.get("text", "") for p in c if isinstance(p, dict))
    text = _TOKEN.findall(c or "")
    calls: List[str] = []
    for tc in message.get("tool_calls") or []:
        fn = tc.get("function") or {}
        args = fn.get("arguments")
        calls += _TOKEN.findall(f"{fn.get('name', '')} {args if isinstance(args, str) else json.dumps(args, sort_keys=True)}")
    return {"text": _shingles(text), "calls": _shingles(calls), "both": _shingles(text + calls)}


def jaccard(a: Set[int], b: Set[int]) -> float:
    if not a or not b:
        return 0.0
    return len(a & b) / len(a | b)


@dataclass
class LoopState:
    kind: str = "none"          # none | hint | suppress
    run_length: int = 0
    score: float = 0.0
    channel: Optional[str] = None


def detect(signatures_newest_first: Sequence[Dict[str, Set[int]]]) -> LoopState:
    sigs = [s for s in signatures_newest_first if any(s[c] for c in CHANNELS)][:MAX_SIGNATURES]
    if len(sigs) < 3:
        return LoopState()
    best = LoopState()
    for ch in CHANNELS:
        run, score = 1, 0.0
        for a, b in zip(sigs, sigs[1:]):
            j = jaccard(a[ch], b[ch])
            if j < MODERATE_SIMILARITY:
                break
            run += 1
            score = max(score, j)
        if run >= 2 and (run, score) > (best.run_length, best.score):
            best = LoopState("none", run, score, ch)
    if best.run_length >= 4 or (best.run_length == 3 and best.score >= HIGH_SIMILARITY):
        best.kind = "suppress"
    elif best.run_length == 3 or (best.run_length == 2 and best.score >= HIGH_SIMILARITY):
        best.kind = "hint"
    else:
        return LoopState()
    return best


@dataclass
class LoopVerdict:
    state: LoopState
    bias: float = 0.0           # added to the tool-call opener's logit (<= 0)
    mask: bool = False          # the opener is forbidden this turn
    reason: str = ""


def _tool_results_after(messages: Sequence[dict], idx: int) -> List[str]:
    out = []
    for m in messages[idx + 1:]:
        if m.get("role") != "tool":
            break
        out.append(str(m.get("content")))
    return out


def check_loops(messages: Sequence[dict], tools_active: bool) -> LoopVerdict:
    idx = [i for i, m in enumerate(messages) if m.get("role") == "assistant"]
    sigs = [signature(messages[i]) for i in reversed(idx)]
    st = detect(sigs)
    if st.kind == "none" or not tools_active:
        return LoopVerdict(st)
    bias = -2.0 * (st.run_length - 1)
    if st.kind == "hint":
        return LoopVerdict(st, bias, False, "soft bias against another tool call")
    recent = list(reversed(idx))[:st.run_length]
    results = [_tool_results_after(messages, i) for i in recent]
    flat = [r for rs in results for r in rs]
    all_failed = bool(flat) and all(re.search(r"\b(error|failed|exception|traceback|not found)\b", r, re.I) for r in flat)
    progressing = len({json.dumps(rs) for rs in results if rs}) > 1
    if os.environ.get("METRALE_LOOP_NO_SUPPRESS") == "1":
        return LoopVerdict(st, bias, False, "suppression disabled by METRALE_LOOP_NO_SUPPRESS")
    if all_failed:
        return LoopVerdict(st, bias, False, "every repeated call failed: the retry stays possible")
    if progressing:
        return LoopVerdict(st, bias, False, "tool results still change between rounds")
    return LoopVerdict(st, bias, True, "tool-call opener masked for this turn")
