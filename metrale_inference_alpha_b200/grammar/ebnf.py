"""EBNF text -> grammar IR. Accepts the GBNF / XGrammar dialect:

    root  ::= "{" ws pair ("," ws pair)* "}"
    pair  ::= string ":" ws value          # comments run to the end of the line
    digit ::= [0-9]   other ::= [^a-z"\\]   any ::= .
    quantifiers: *  +  ?  {n}  {n,}  {n,m}

A rule body ends where the next ``name ::=`` begins, so bodies may span lines.
Role of the reference's ``crates/grammar/src/grammar`` parser.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from .ir import MAX_CP, GrammarError

_NAME_START = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ_"
_NAME_REST = _NAME_START + "0123456789-."
_ESC = {"n": 10, "t": 9, "r": 13, "0": 0, "\\": 92, '"': 34, "'": 39, "[": 91, "]": 93, "-": 45, "^": 94, "/": 47}


class _P:
    def __init__(self, text: str):
        self.s, self.i = text, 0

    def err(self, msg: str):
        line = self.s.count("\n", 0, self.i) + 1
        raise GrammarError(f"EBNF line {line}: {msg}")

    def ws(self) -> None:
        s = self.s
        while self.i < len(s):
            c = s[self.i]
            if c in " \t\r\n":
                self.i += 1
            elif c == "#":
                while self.i < len(s) and s[self.i] != "\n":
                    self.i += 1
            else:
                break

    def peek(self) -> str:
        return self.s[self.i] if self.i < len(self.s) else ""

    def name(self) -> str:
        j = self.i
        if self.peek() not in _NAME_START or not self.peek():
            self.err("rule name expected")
        while self.i < len(self.s) and self.s[self.i] in _NAME_REST:
            self.i += 1
        return self.s[j:self.i]

    def at_rule_start(self) -> bool:
        """Is the cursor at ``name ::=``?"""
        j = self.i
        if j >= len(self.s) or self.s[j] not in _NAME_START:
            return False
        while j < len(self.s) and self.s[j] in _NAME_REST:
            j += 1
        while j < len(self.s) and self.s[j] in " \t":
            j += 1
        return self.s.startswith("::=", j)

    def escape(self) -> int:
        """Cursor is after a backslash; returns the code point."""
        c = self.peek()
        if not c:
            self.err("dangling backslash")
        self.i += 1
        if c in _ESC:
            return _ESC[c]
        n = {"x": 2, "u": 4, "U": 8}.get(c)
        if n is None:
            self.err(f"unknown escape \\{c}")
        h = self.s[self.i:self.i + n]
        if len(h) != n:
            self.err("short hex escape")
        try:
            v = int(h, 16)
        except ValueError:
            self.err("bad hex escape")
        self.i += n
        if v > MAX_CP:
            self.err("escape beyond U+10FFFF")
        return v

    def string(self) -> tuple:
        q = self.peek()
        self.i += 1
        out = bytearray()
        while True:
            c = self.peek()
            if not c or c == "\n":
                self.err("unterminated string")
            self.i += 1
            if c == q:
                break
            if c == "\\":
                cp = self.escape()
                out += bytes([cp]) if cp < 0x80 else chr(cp).encode("utf-8", "surrogatepass")
            else:
                out += c.encode("utf-8")
        return ("lit", bytes(out)) if out else ("empty",)

    def char_class(self) -> tuple:
        self.i += 1                     # [
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
            lo = self.escape() if c == "\\" else ord(c)
            hi = lo
            if self.peek() == "-" and self.s[self.i + 1:self.i + 2] not in ("]", ""):
                self.i += 1
                d = self.peek()
                self.i += 1
                hi = self.escape() if d == "\\" else ord(d)
                if hi < lo:
                    self.err("reversed range in character class")
            ranges.append((lo, hi))
        return ("cls", ranges, neg)

    def quantifier(self, e: tuple) -> tuple:
        while True:
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
                if j < 0:
                    self.err("unterminated {}")
                body = self.s[self.i + 1:j].replace(" ", "")
                self.i = j + 1
                try:
                    if "," in body:
                        a, b = body.split(",", 1)
                        lo, hi = int(a or 0), (int(b) if b else None)
                    else:
                        lo = hi = int(body)
                except ValueError:
                    self.err("bad repetition count")
                if lo < 0 or (hi is not None and (hi < lo or hi > 100000)):
                    self.err("bad repetition range")
                e = ("rep", e, lo, hi)
            else:
                return e

    def atom(self) -> tuple:
        c = self.peek()
        if c in "\"'":
            return self.string()
        if c == "[":
            return self.char_class()
        if c == ".":
            self.i += 1
            return ("cls", [(0, MAX_CP)], False)
        if c == "(":
            self.i += 1
            e = self.alternation()
            self.ws()
            if self.peek() != ")":
                self.err("')' expected")
            self.i += 1
            return e
        if c and c in _NAME_START:
            return ("ref", self.name())
        self.err(f"unexpected {c!r}" if c else "unexpected end of grammar")

    def sequence(self) -> tuple:
        items = []
        while True:
            self.ws()
            c = self.peek()
            if not c or c in "|)" or self.at_rule_start():
                break
            items.append(self.quantifier(self.atom()))
        if not items:
            return ("empty",)
        return items[0] if len(items) == 1 else ("seq", items)

    def alternation(self) -> tuple:
        alts = [self.sequence()]
        while True:
            self.ws()
            if self.peek() != "|":
                break
            self.i += 1
            alts.append(self.sequence())
        return alts[0] if len(alts) == 1 else ("alt", alts)


def parse_ebnf(text: str) -> Dict[str, tuple]:
    p = _P(text)
    rules: Dict[str, tuple] = {}
    p.ws()
    while p.i < len(p.s):
        name = p.name()
        p.ws()
        if not p.s.startswith("::=", p.i):
            p.err("'::=' expected")
        p.i += 3
        if name in rules:
            p.err(f"rule '{name}' defined twice")
        rules[name] = p.alternation()
        p.ws()
        if p.peek() == ")":
            p.err("unbalanced ')'")
    if not rules:
        raise GrammarError("empty grammar")
    return rules
