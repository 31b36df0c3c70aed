"""Structural tags: unconstrained text in which a trigger string switches to a constrained
segment (how tool calls are forced to be well-formed while the rest of the answer stays free).

The free text is the Aho-Corasick automaton of the triggers written as right-recursive rules
(one rule per automaton state; the matcher elides the frame of a tail call, so the stack does not
grow with the text). The byte that would complete a trigger enters that trigger's tag rule
instead: the rest of ``begin``, the body, ``end``; then the automaton restarts.

Role of the reference's ``crates/grammar/src/structural_tag``.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

from .ebnf import parse_ebnf
from .ir import GrammarError
from .regex import parse_regex
from .schema import base_rules, schema_to_rules


def rename_rules(rules: Dict[str, tuple], keep: set, prefix: str) -> Dict[str, tuple]:
    def ren(e):
        k = e[0]
        if k == "ref":
            return e if e[1] in keep else ("ref", prefix + e[1])
        if k in ("seq", "alt"):
            return (k, [ren(x) for x in e[1]])
        if k == "rep":
            return ("rep", ren(e[1]), e[2], e[3])
        return e
    return {(n if n in keep else prefix + n): ren(b) for n, b in rules.items()}


def _automaton(triggers: Sequence[bytes]):
    """Aho-Corasick as a full DFA: delta[state][byte] -> state, hit[state] -> trigger index or -1."""
    goto: List[Dict[int, int]] = [{}]
    hit: List[int] = [-1]
    for ti, t in enumerate(triggers):
        s = 0
        for c in t:
            if c not in goto[s]:
                goto.append({})
                hit.append(-1)
                goto[s][c] = len(goto) - 1
            s = goto[s][c]
        if hit[s] < 0:
            hit[s] = ti
    fail = [0] * len(goto)
    delta = [[0] * 256 for _ in goto]
    order = []
    for c in range(256):
        t = goto[0].get(c)
        if t is not None:
            delta[0][c] = t
            order.append(t)
    i = 0
    while i < len(order):
        s = order[i]
        i += 1
        if hit[s] < 0:
            hit[s] = hit[fail[s]]
        for c in range(256):
            t = goto[s].get(c)
            if t is not None:
                fail[t] = delta[fail[s]][c]
                delta[s][c] = t
                order.append(t)
            else:
                delta[s][c] = delta[fail[s]][c]
    return delta, hit


def structural_tag_rules(tags: Sequence[dict], triggers: Sequence[str], at_least_one: bool = False,
                         stop_after_first: bool = False, calls_only: bool = False) -> Dict[str, tuple]:
    if not triggers:
        raise GrammarError("structural tag needs at least one trigger")
    trig = [t.encode("utf-8") for t in triggers]
    if any(not t for t in trig):
        raise GrammarError("empty trigger")
    for a in trig:
        for b in trig:
            if a is not b and a in b:
                raise GrammarError("a trigger may not occur inside another trigger")
    rules: Dict[str, tuple] = dict(base_rules())
    keep = set(rules.keys())
    per_trigger: List[List[tuple]] = [[] for _ in trig]
    for i, tag in enumerate(tags):
        begin = tag.get("begin", "").encode("utf-8")
        end = tag.get("end", "").encode("utf-8")
        owner = [j for j, t in enumerate(trig) if begin.startswith(t)]
        if not owner:
            raise GrammarError(f"tag {i}: 'begin' starts with none of the triggers")
        j = owner[0]
        prefix = f"t{i}."
        if "grammar" in tag:
            sub = rename_rules(parse_ebnf(tag["grammar"]), set(), prefix)
            body = ("ref", prefix + "root")
        elif "regex" in tag:
            sub, body = {}, parse_regex(tag["regex"])
        else:
            sub = rename_rules(schema_to_rules(tag.get("schema", True), root="root"), keep, prefix)
            body = ("ref", prefix + "root")
        rules.update(sub)
        rest = begin[len(trig[j]):]
        seq = ([("lit", rest)] if rest else []) + [body] + ([("lit", end)] if end else [])
        per_trigger[j].append(seq[0] if len(seq) == 1 else ("seq", seq))
    for j, alts in enumerate(per_trigger):
        if not alts:
            raise GrammarError(f"trigger {triggers[j]!r} has no tag")
        rules[f"tag.{j}"] = alts[0] if len(alts) == 1 else ("alt", alts)
    if calls_only:
        # no free text at all: one tagged segment, then (unless stop_after_first) more of them
        # separated by white space
        one = ("alt", [("seq", [("lit", t), ("ref", f"tag.{j}")]) for j, t in enumerate(trig)])
        rules["call"] = one
        more = ("empty",) if stop_after_first else ("rep", ("seq", [("ref", "ws"), ("ref", "call")]), 0, None)
        rules["root"] = ("seq", [("ref", "ws"), ("ref", "call"), more, ("ref", "ws")])
        return rules
    delta, hit = _automaton(trig)
    live = [s for s in range(len(delta)) if hit[s] < 0]

    def automaton(name: str, may_end: bool, after: tuple) -> None:
        for s in live:
            alts: List[tuple] = []
            c = 0
            while c < 256:
                t = delta[s][c]
                d = c
                while d + 1 < 256 and delta[s][d + 1] == t and hit[t] < 0:
                    d += 1
                if hit[t] >= 0:
                    alts.append(("seq", [("bytes", c, c), ("ref", f"tag.{hit[t]}"), after]))
                    d = c
                else:
                    alts.append(("seq", [("bytes", c, d), ("ref", f"{name}.{t}")]))
                c = d + 1
            if may_end:
                alts.append(("empty",))
            rules[f"{name}.{s}"] = ("alt", alts)

    if stop_after_first:
        after = ("empty",)
    else:
        after = ("ref", "free.0")
        automaton("free", True, after)
    if at_least_one or stop_after_first:
        automaton("first", not at_least_one, after)
        rules["root"] = ("ref", "first.0")
    else:
        rules["root"] = ("ref", "free.0")
    return rules
