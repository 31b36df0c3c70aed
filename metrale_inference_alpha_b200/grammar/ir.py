"""Grammar IR and its compiled form.

A grammar is a set of named rules over bytes. Rule bodies are expression tuples:

    ("empty",)                       the empty string
    ("lit", bytes)                   a literal byte string
    ("cls", ranges, negated)         one character; ranges are inclusive code-point pairs
    ("ref", name)                    another rule
    ("seq", [e, ...])  ("alt", [e, ...])
    ("rep", e, lo, hi)               lo..hi repetitions (hi None = unbounded)
    ("bytes", lo, hi)                one raw byte in lo..hi

``compile_rules`` turns every rule into a Thompson NFA whose edges are byte ranges, rule
references or epsilons, flattened into integer arrays that both the Python matcher
(``grammar/matcher.py``) and the C++ one (``native/grammar_pda.cpp``) walk. Characters outside
ASCII are expanded to UTF-8 byte-range sequences, so the matcher itself only ever sees bytes and
a token may end in the middle of a character.

Role of the reference's ``crates/grammar/src/{grammar,compiler,fsm}``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

EDGE_EPS, EDGE_BYTES, EDGE_RULE = 0, 1, 2
MAX_CP = 0x10FFFF
_MAX_NODES = 2_000_000


class GrammarError(ValueError):
    pass


# ------------------------------------------------------------------ UTF-8 range expansion
def _encode(cp: int) -> bytes:
    return chr(cp).encode("utf-8", "surrogatepass")


def _split_same_len(lo: int, hi: int, out: List[List[Tuple[int, int]]]) -> None:
    """[lo, hi] encode to the same number of bytes: cut it until every piece is a product of
    per-byte ranges."""
    n = len(_encode(lo))
    for i in range(1, n):
        m = (1 << (6 * i)) - 1
        if (lo & ~m) != (hi & ~m):
            if (lo & m) != 0:
                _split_same_len(lo, lo | m, out)
                _split_same_len((lo | m) + 1, hi, out)
                return
            if (hi & m) != m:
                _split_same_len(lo, (hi & ~m) - 1, out)
                _split_same_len(hi & ~m, hi, out)
                return
    a, b = _encode(lo), _encode(hi)
    out.append([(x, y) for x, y in zip(a, b)])


def utf8_sequences(lo: int, hi: int) -> List[List[Tuple[int, int]]]:
    """Byte-range sequences that together accept exactly the UTF-8 encodings of [lo, hi]
    (surrogates removed)."""
    out: List[List[Tuple[int, int]]] = []
    pieces = []
    if lo <= 0xD7FF and hi >= 0xE000:
        pieces = [(lo, 0xD7FF), (0xE000, hi)]
    elif 0xD800 <= lo <= 0xDFFF or 0xD800 <= hi <= 0xDFFF:
        lo2 = 0xE000 if 0xD800 <= lo <= 0xDFFF else lo
        hi2 = 0xD7FF if 0xD800 <= hi <= 0xDFFF else hi
        pieces = [(lo2, hi2)] if lo2 <= hi2 else []
    else:
        pieces = [(lo, hi)]
    for a, b in pieces:
        for edge in (0x7F, 0x7FF, 0xFFFF):
            if a <= edge < b:
                _split_same_len(a, edge, out)
                a = edge + 1
        _split_same_len(a, b, out)
    return out


def normalize_ranges(ranges: Sequence[Tuple[int, int]], negated: bool = False) -> List[Tuple[int, int]]:
    rs = sorted((max(0, a), min(MAX_CP, b)) for a, b in ranges if a <= b)
    merged: List[Tuple[int, int]] = []
    for a, b in rs:
        if merged and a <= merged[-1][1] + 1:
            merged[-1] = (merged[-1][0], max(merged[-1][1], b))
        else:
            merged.append((a, b))
    if not negated:
        return merged
    out, prev = [], 0
    for a, b in merged:
        if a > prev:
            out.append((prev, a - 1))
        prev = b + 1
    if prev <= MAX_CP:
        out.append((prev, MAX_CP))
    return out


# ------------------------------------------------------------------ compiled form
@dataclass
class CompiledGrammar:
    edge_begin: List[int]            # per node: first edge; n_nodes + 1 entries
    edge_kind: List[int]
    edge_a: List[int]                # BYTES: lo byte; RULE: rule index
    edge_b: List[int]                # BYTES: hi byte
    edge_to: List[int]
    final: List[int]                 # per node: bit 0 = the rule may end here; bit 1 = nothing but
                                     # the end can follow (a call returning here is a tail call)
    rule_start: List[int]
    rule_names: List[str]
    root: int
    key: str = ""                    # cache key of the source it was compiled from
    _native: object = field(default=None, repr=False, compare=False)

    @property
    def n_nodes(self) -> int:
        return len(self.final)

    def __getstate__(self):                # the native tables are rebuilt where the copy lands
        d = dict(self.__dict__)
        d["_native"] = None
        return d


class _Builder:
    def __init__(self):
        self.edges: List[List[Tuple[int, int, int, int]]] = []
        self.final: List[int] = []

    def node(self) -> int:
        if len(self.edges) >= _MAX_NODES:
            raise GrammarError("grammar too large")
        self.edges.append([])
        self.final.append(0)
        return len(self.edges) - 1

    def edge(self, a: int, kind: int, x: int, y: int, b: int) -> None:
        self.edges[a].append((kind, x, y, b))

    # returns the exit node of the fragment that starts at `s`
    def build(self, e, s: int, rules: Dict[str, int]) -> int:
        k = e[0]
        if k == "empty":
            return s
        if k == "lit":
            for c in e[1]:
                t = self.node()
                self.edge(s, EDGE_BYTES, c, c, t)
                s = t
            return s
        if k == "bytes":                  # raw byte range (may cut through UTF-8 sequences)
            t = self.node()
            self.edge(s, EDGE_BYTES, e[1], e[2], t)
            return t
        if k == "cls":
            rs = normalize_ranges(e[1], e[2])
            if not rs:
                return self.node()         # unreachable exit: matches nothing
            t = self.node()
            for lo, hi in rs:
                if hi <= 0x7F:
                    self.edge(s, EDGE_BYTES, lo, hi, t)
                    continue
                if lo <= 0x7F:
                    self.edge(s, EDGE_BYTES, lo, 0x7F, t)
                    lo = 0x80
                for seq in utf8_sequences(lo, hi):
                    cur = s
                    for i, (x, y) in enumerate(seq):
                        nxt = t if i == len(seq) - 1 else self.node()
                        self.edge(cur, EDGE_BYTES, x, y, nxt)
                        cur = nxt
            return t
        if k == "ref":
            if e[1] not in rules:
                raise GrammarError(f"undefined rule '{e[1]}'")
            t = self.node()
            self.edge(s, EDGE_RULE, rules[e[1]], 0, t)
            return t
        if k == "seq":
            for x in e[1]:
                s = self.build(x, s, rules)
            return s
        if k == "alt":
            t = self.node()
            for x in e[1]:
                a = self.node()
                self.edge(s, EDGE_EPS, 0, 0, a)
                self.edge(self.build(x, a, rules), EDGE_EPS, 0, 0, t)
            return t
        if k == "rep":
            _, x, lo, hi = e
            if hi is not None and hi < lo:
                raise GrammarError("repetition with max < min")
            for _ in range(lo):
                s = self.build(x, s, rules)
            if hi is None:
                # loop: s -> body -> back to s; exit through t
                a, t = self.node(), self.node()
                self.edge(s, EDGE_EPS, 0, 0, a)
                self.edge(s, EDGE_EPS, 0, 0, t)
                z = self.build(x, a, rules)
                self.edge(z, EDGE_EPS, 0, 0, a)
                self.edge(z, EDGE_EPS, 0, 0, t)
                return t
            t = self.node()
            self.edge(s, EDGE_EPS, 0, 0, t)
            for _ in range(hi - lo):
                s = self.build(x, s, rules)
                self.edge(s, EDGE_EPS, 0, 0, t)
            return t
        raise GrammarError(f"unknown expression kind {k!r}")


# ------------------------------------------------------------------ rule-level checks + flatten
def _nullable_and_left(rules: Dict[str, tuple]) -> None:
    """Refuses left recursion (a rule that can reach itself without consuming a byte): the
    pushdown closure would never terminate on it."""
    nullable: Dict[str, bool] = {n: False for n in rules}

    def null(e) -> bool:
        k = e[0]
        if k == "empty":
            return True
        if k == "lit":
            return len(e[1]) == 0
        if k == "cls":
            return False
        if k == "ref":
            return nullable.get(e[1], False)
        if k == "seq":
            return all(null(x) for x in e[1])
        if k == "alt":
            return any(null(x) for x in e[1])
        if k == "rep":
            return e[2] == 0 or null(e[1])
        return False

    changed = True
    while changed:
        changed = False
        for n, body in rules.items():
            v = null(body)
            if v and not nullable[n]:
                nullable[n], changed = True, True

    def left(e, acc: set) -> None:
        k = e[0]
        if k == "ref":
            acc.add(e[1])
        elif k == "seq":
            for x in e[1]:
                left(x, acc)
                if not null(x):
                    break
        elif k == "alt":
            for x in e[1]:
                left(x, acc)
        elif k == "rep":
            left(e[1], acc)

    graph = {}
    for n, body in rules.items():
        s: set = set()
        left(body, s)
        graph[n] = s
    state: Dict[str, int] = {}

    def visit(n: str, path: List[str]) -> None:
        if state.get(n) == 2 or n not in graph:
            return
        if state.get(n) == 1:
            raise GrammarError("left recursion through " + " -> ".join(path + [n]))
        state[n] = 1
        for m in graph[n]:
            visit(m, path + [n])
        state[n] = 2

    import sys
    old = sys.getrecursionlimit()
    sys.setrecursionlimit(max(old, 10000))
    try:
        for n in rules:
            visit(n, [])
    finally:
        sys.setrecursionlimit(old)


def compile_rules(rules: Dict[str, tuple], root: str = "root", key: str = "") -> CompiledGrammar:
    if root not in rules:
        raise GrammarError(f"no '{root}' rule")
    _nullable_and_left(rules)
    # only rules reachable from the root are compiled
    order: List[str] = []
    seen = set()

    def refs(e, acc):
        if e[0] == "ref":
            acc.append(e[1])
        elif e[0] in ("seq", "alt"):
            for x in e[1]:
                refs(x, acc)
        elif e[0] == "rep":
            refs(e[1], acc)

    todo = [root]
    while todo:
        n = todo.pop()
        if n in seen:
            continue
        if n not in rules:
            raise GrammarError(f"undefined rule '{n}'")
        seen.add(n)
        order.append(n)
        acc: List[str] = []
        refs(rules[n], acc)
        todo.extend(acc)
    index = {n: i for i, n in enumerate(order)}
    b = _Builder()
    starts = []
    for n in order:
        s = b.node()
        starts.append(s)
        z = b.build(rules[n], s, index)
        b.final[z] = 1
    # tail nodes: everything reachable is epsilon edges ending in a final node
    n_nodes = len(b.edges)
    only_eps = [all(k == EDGE_EPS for (k, _, _, _) in es) for es in b.edges]
    for n in range(n_nodes):
        if not only_eps[n]:
            continue
        seen_n, todo_n, ok, fin = {n}, [n], True, False
        while todo_n and ok:
            m = todo_n.pop()
            fin = fin or bool(b.final[m] & 1)
            for (_, _, _, t) in b.edges[m]:
                if not only_eps[t]:
                    ok = False
                    break
                if t not in seen_n:
                    seen_n.add(t)
                    todo_n.append(t)
        if ok and fin:
            b.final[n] |= 2
    edge_begin, kind, ea, eb, to = [0], [], [], [], []
    for es in b.edges:
        for (k, x, y, t) in es:
            kind.append(k)
            ea.append(x)
            eb.append(y)
            to.append(t)
        edge_begin.append(len(kind))
    return CompiledGrammar(edge_begin, kind, ea, eb, to, b.final, starts, order, 0, key)
