"""Regular expression -> grammar IR (full-match semantics: the output must match the whole
pattern). Supported: literals, ``.``, classes with ranges and ``\\d \\w \\s \\D \\W \\S``, groups
(capturing, ``(?:...)``, named), alternation, ``* + ? {m} {m,} {m,n}`` (a lazy or possessive
suffix is accepted and ignored: it does not change the language), ``^`` / ``$`` at the ends.
Back-references and look-around change the language class and are refused.

Role of the reference's ``crates/grammar/src/regex``.
"""
from __future__ import annotations

from typing import List, Tuple

from .ir import MAX_CP, GrammarError

_D = [(48, 57)]
_W = [(48, 57), (65, 90), (95, 95), (97, 122)]
_S = [(9, 13), (32, 32)]
_SIMPLE = {"n": 10, "t": 9, "r": 13, "f": 12, "v": 11, "0": 0, "a": 7, "e": 27}


def _negate(rs):
    from .ir import normalize_ranges
    return normalize_ranges(rs, True)


class _R:
    def __init__(self, pat: str):
        self.s, self.i = pat, 0

    def err(self, msg):
        raise GrammarError(f"regex at {self.i}: {msg}")

    def peek(self) -> str:
        return self.s[self.i] if self.i < len(self.s) else ""

    def hexn(self, n: int) -> int:
        h = self.s[self.i:self.i + n]
        if len(h) != n:
            self.err("short hex escape")
        try:
            v = int(h, 16)
        except ValueError:
            self.err("bad hex escape")
        self.i += n
        return v

    def escape(self, in_class: bool):
        """After a backslash. Returns ("cp", code point) or ("set", ranges)."""
        c = self.peek()
        if not c:
            self.err("dangling backslash")
        self.i += 1
        if c == "d":
            return ("set", _D)
        if c == "D":
            return ("set", _negate(_D))
        if c == "w":
            return ("set", _W)
        if c == "W":
            return ("set", _negate(_W))
        if c == "s":
            return ("set", _S)
        if c == "S":
            return ("set", _negate(_S))
        if c in _SIMPLE:
            return ("cp", _SIMPLE[c])
        if c == "x":
            if self.peek() == "{":
                j = self.s.find("}", self.i)
                if j < 0:
                    self.err("unterminated \\x{")
                try:
                    v = int(self.s[self.i + 1:j], 16)
                except ValueError:
                    self.err("bad hex escape")
                self.i = j + 1
                return ("cp", v)
            return ("cp", self.hexn(2))
        if c == "u":
            return ("cp", self.hexn(4))
        if c == "U":
            return ("cp", self.hexn(8))
        if c in "bBAZzG" and not in_class:
            self.err(f"\\{c} assertions are not supported")
        if c == "b" and in_class:
            return ("cp", 8)
        if c.isdigit() or c == "k":
            self.err("back-references are not supported")
        if c in "pP":
            self.err("unicode property classes are not supported")
        return ("cp", ord(c))

    def char_class(self) -> tuple:
        self.i += 1
        neg = self.peek() == "^"
        if neg:
            self.i += 1
        ranges: List[Tuple[int, int]] = []
        first = True
        while True:
            c = self.peek()
            if not c:
                self.err("unterminated character class")
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            self.i += 1
            if c == "\\":
                k, v = self.escape(True)
                if k == "set":
                    ranges += v
                    continue
                lo = v
            else:
                lo = ord(c)
            hi = lo
            if self.peek() == "-" and self.s[self.i + 1:self.i + 2] not in ("]", ""):
                self.i += 1
                d = self.peek()
                self.i += 1
                if d == "\\":
                    k, v = self.escape(True)
                    if k == "set":
                        self.err("class shorthand as a range end")
                    hi = v
                else:
                    hi = ord(d)
                if hi < lo:
                    self.err("reversed range")
            ranges.append((lo, hi))
        return ("cls", ranges, neg)

    def quant(self, e: tuple) -> tuple:
        c = self.peek()
        if c == "*":
            self.i += 1
            e = ("rep", e, 0, None)
        elif c == "+":
            self.i += 1
            e = ("rep", e, 1, None)
        elif c == "?":
            self.i += 1
            e = ("rep", e, 0, 1)
        elif c == "{":
            j = self.s.find("}", self.i)
            body = self.s[self.i + 1:j] if j > 0 else ""
            ok = j > 0 and body.replace(",", "", 1).replace(" ", "").isdigit() and body[:1].isdigit()
            if not ok:
                return e                      # a literal brace, as in most engines
            self.i = j + 1
            if "," in body:
                a, b = body.split(",", 1)
                lo, hi = int(a), (int(b) if b.strip() else None)
            else:
                lo = hi = int(body)
            if hi is not None and (hi < lo or hi > 100000):
                self.err("bad repetition range")
            e = ("rep", e, lo, hi)
        else:
            return e
        if self.peek() in ("?", "+"):         # lazy / possessive: same language
            self.i += 1
        return e

    def atom(self):
        c = self.peek()
        self.i += 1
        if c == "(":
            if self.s.startswith("?:", self.i):
                self.i += 2
            elif self.s.startswith("?P<", self.i) or (self.s.startswith("?<", self.i)
                                                      and self.s[self.i + 2:self.i + 3] not in ("=", "!")):
                j = self.s.find(">", self.i)
                if j < 0:
                    self.err("unterminated group name")
                self.i = j + 1
            elif self.peek() == "?":
                self.err("look-around and inline flags are not supported")
            e = self.alt()
            if self.peek() != ")":
                self.err("')' expected")
            self.i += 1
            return e
        if c == "[":
            self.i -= 1
            return self.char_class()
        if c == ".":
            return ("cls", [(10, 10)], True)
        if c == "\\":
            k, v = self.escape(False)
            if k == "set":
                return ("cls", v, False)
            return ("lit", chr(v).encode("utf-8", "surrogatepass"))
        if c in "*+?":
            self.err("nothing to repeat")
        return ("lit", c.encode("utf-8"))

    def seq(self) -> tuple:
        items = []
        while self.i < len(self.s) and self.peek() not in "|)":
            c = self.peek()
            if c == "^":
                if items:
                    self.err("'^' inside the pattern is not supported")
                self.i += 1
                continue
            if c == "$":
                rest = self.s[self.i + 1:self.i + 2]
                if rest not in ("", "|", ")"):
                    self.err("'$' inside the pattern is not supported")
                self.i += 1
                continue
            items.append(self.quant(self.atom()))
        # merge neighbouring literals
        merged: List[tuple] = []
        for e in items:
            if e[0] == "lit" and merged and merged[-1][0] == "lit":
                merged[-1] = ("lit", merged[-1][1] + e[1])
            else:
                merged.append(e)
        if not merged:
            return ("empty",)
        return merged[0] if len(merged) == 1 else ("seq", merged)

    def alt(self) -> tuple:
        alts = [self.seq()]
        while self.peek() == "|":
            self.i += 1
            alts.append(self.seq())
        return alts[0] if len(alts) == 1 else ("alt", alts)


def parse_regex(pattern: str) -> tuple:
    p = _R(pattern)
    e = p.alt()
    if p.i != len(p.s):
        p.err("unbalanced ')'")
    return e
