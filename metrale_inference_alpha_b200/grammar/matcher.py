"""Pushdown matcher over a ``CompiledGrammar`` (pure Python: the oracle for the C++ matcher in
``native/grammar_pda.cpp`` and the fallback when the native runtime is not built).

State is a set of items ``(node, frame)``; a frame is an interned ``(return node, parent frame)``
pair, so the many stacks of an ambiguous parse share their tails. ``feed`` is atomic: either
every byte is accepted and the state advances, or the state is unchanged.

Role of the reference's ``crates/grammar/src/matcher``.
"""
from __future__ import annotations

from typing import Dict, FrozenSet, List, Optional, Set, Tuple

from .ir import EDGE_BYTES, EDGE_EPS, EDGE_RULE, CompiledGrammar

Item = Tuple[int, int]
ROOT_FRAME = -1


class GrammarMatcher:
    def __init__(self, g: CompiledGrammar):
        self.g = g
        self.frames: List[Tuple[int, int]] = []
        self._intern: Dict[Tuple[int, int], int] = {}
        self.items: FrozenSet[Item] = self._closure({(g.rule_start[g.root], ROOT_FRAME)})
        self._history: List[FrozenSet[Item]] = []

    def _frame(self, ret: int, parent: int) -> int:
        k = (ret, parent)
        f = self._intern.get(k)
        if f is None:
            f = len(self.frames)
            self.frames.append(k)
            self._intern[k] = f
        return f

    def _closure(self, seed: Set[Item]) -> FrozenSet[Item]:
        g = self.g
        out: Set[Item] = set()
        todo = list(seed)
        while todo:
            it = todo.pop()
            if it in out:
                continue
            out.add(it)
            n, f = it
            for e in range(g.edge_begin[n], g.edge_begin[n + 1]):
                k = g.edge_kind[e]
                if k == EDGE_EPS:
                    todo.append((g.edge_to[e], f))
                elif k == EDGE_RULE:
                    t = g.edge_to[e]
                    # tail call: returning to `t` could only end the caller, so reuse its frame
                    todo.append((g.rule_start[g.edge_a[e]], f if g.final[t] & 2 else self._frame(t, f)))
            if g.final[n] & 1 and f != ROOT_FRAME:
                ret, parent = self.frames[f]
                todo.append((ret, parent))
        return frozenset(out)

    def _step(self, items: FrozenSet[Item], c: int) -> FrozenSet[Item]:
        g = self.g
        nxt: Set[Item] = set()
        for n, f in items:
            for e in range(g.edge_begin[n], g.edge_begin[n + 1]):
                if g.edge_kind[e] == EDGE_BYTES and g.edge_a[e] <= c <= g.edge_b[e]:
                    nxt.add((g.edge_to[e], f))
        return self._closure(nxt) if nxt else frozenset()

    # ------------------------------------------------------------------ public
    def feed_bytes(self, bs: bytes) -> bool:
        items = self.items
        for c in bs:
            items = self._step(items, c)
            if not items:
                return False
        self.items = items
        return True

    def accepts(self, bs: bytes) -> bool:
        """Would `bs` be accepted from the current state (state unchanged)?"""
        items = self.items
        for c in bs:
            items = self._step(items, c)
            if not items:
                return False
        return True

    def is_complete(self) -> bool:
        return any(f == ROOT_FRAME and self.g.final[n] & 1 for n, f in self.items)

    def can_continue(self) -> bool:
        """False when the only legal continuation is to stop."""
        g = self.g
        return any(g.edge_kind[e] == EDGE_BYTES for n, _ in self.items
                   for e in range(g.edge_begin[n], g.edge_begin[n + 1]))

    def push(self) -> None:
        self._history.append(self.items)

    def rollback(self, n: int) -> None:
        for _ in range(n):
            self.items = self._history.pop()

    def clone(self) -> "GrammarMatcher":
        m = GrammarMatcher.__new__(GrammarMatcher)
        m.g, m.frames, m._intern = self.g, list(self.frames), dict(self._intern)
        m.items, m._history = self.items, list(self._history)
        return m


def matches(g: CompiledGrammar, data: bytes) -> bool:
    m = GrammarMatcher(g)
    return m.feed_bytes(data) and m.is_complete()


class TokenMatcher:
    """Token-level adapter with the interface the sampler uses (``allowed_mask`` / ``advance`` /
    ``rollback``). Uses the native matcher when it is built, else this module's."""

    def __init__(self, grammar: CompiledGrammar, tokenizer, eos_token_id: Optional[int] = None,
                 vocab_size: Optional[int] = None, prefer_native: bool = True):
        self.g, self.tk, self.eos = grammar, tokenizer, eos_token_id
        self.n = vocab_size or tokenizer.vocab_size
        self._history: List[int] = []
        self._native = None
        if prefer_native:
            from .. import native
            if native.available() and native.has_pda():
                self._native = native.NativePda(grammar, tokenizer, self.n)
        self._py = None if self._native is not None else GrammarMatcher(grammar)
        self._bytes: Optional[List[bytes]] = None

    # a copy sent to another rank is rebuilt by replaying the accepted tokens
    def __getstate__(self):
        return {"g": self.g, "tk": self.tk, "eos": self.eos, "n": self.n, "history": list(self._history),
                "native": self._native is not None}

    def __setstate__(self, st):
        self.__init__(st["g"], st["tk"], st["eos"], st["n"], st["native"])
        for t in st["history"]:
            self.advance(t)

    def observe_logits(self, row) -> None:
        pass

    def _token_bytes(self) -> List[bytes]:
        if self._bytes is None:
            self._bytes = [self.tk.token_bytes(t) or b"" for t in range(self.n)]
        return self._bytes

    def allowed_mask(self, vocab: int):
        import torch
        if self._native is not None:
            mask = self._native.fill_mask(vocab, self.eos)
        else:
            mask = torch.zeros(vocab, dtype=torch.bool)
            tb = self._token_bytes()
            first = [bool(self._py._step(self._py.items, c)) for c in range(256)]
            for t in range(min(vocab, self.n)):
                b = tb[t]
                if t == self.eos or not b or not first[b[0]]:
                    continue
                if len(b) == 1 or self._py.accepts(b):
                    mask[t] = True
            if self.eos is not None and self.eos < vocab and self._py.is_complete():
                mask[self.eos] = True
        if not bool(mask.any()) and self.eos is not None and self.eos < vocab:
            mask[self.eos] = True
        return mask

    def advance(self, tid: int) -> None:
        if tid == self.eos:
            return
        if self._native is not None:
            self._native.advance(int(tid))
        else:
            self._py.push()
            self._py.feed_bytes(self.tk.token_bytes(int(tid)) or b"")
        self._history.append(int(tid))

    def rollback(self, n: int) -> None:
        n = min(n, len(self._history))
        if n <= 0:
            return
        if self._native is not None:
            self._native.rollback(n)
        else:
            self._py.rollback(n)
        del self._history[-n:]

    def is_complete(self) -> bool:
        return self._native.is_complete() if self._native is not None else self._py.is_complete()

    def feed_bytes(self, bs: bytes) -> bool:
        return self._native.feed(bs) if self._native is not None else self._py.feed_bytes(bs)
