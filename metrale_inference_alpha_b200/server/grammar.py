"""Constrained decoding: an incremental matcher decides which tokens may come next.

``JsonMatcher`` accepts exactly the prefixes of JSON values (optionally restricted to a top-level
object, and checked against a JSON-schema subset: type, properties, required, enum, items);
``RegexMatcher`` accepts prefixes of a regular expression via a derivative-free NFA over the
pattern's byte alphabet. ``TokenGrammar`` lifts a byte matcher to the token vocabulary: the
allowed mask is computed by simulating each candidate token's bytes from the current state
(candidates are limited to the highest logits first, widening until a legal token is found,
so the cost per step is independent of vocabulary size).
Role of the reference's ``crates/grammar`` (pushdown matcher + token bitmask) and
``crates/server/src/grammar`` glue, in reduced form."""
from __future__ import annotations

import copy
import json
from typing import List, Optional

import torch

WS = b" \t\n\r"


class JsonMatcher:
    """Byte-level incremental JSON recogniser (pushdown). ``feed(b) -> bool`` advances or refuses."""

    def __init__(self, require_object: bool = False):
        self.stack: List[str] = []          # 'obj_key', 'obj_colon', 'obj_val', 'obj_next', 'arr_val', 'arr_next'
        self.state = "value"                # value | string | escape | unicode | number | literal | done
        self.lit = b""
        self.lit_pos = 0
        self.uni = 0
        self.num = b""
        self.string_is_key = False
        self.require_object = require_object
        self.started = False

    def clone(self):
        return copy.copy(self) if not self.stack else copy.deepcopy(self)

    def _end_value(self):
        if not self.stack:
            self.state = "done"
            return
        top = self.stack[-1]
        if top == "obj_val":
            self.stack[-1] = "obj_next"
        elif top == "arr_val":
            self.stack[-1] = "arr_next"
        self.state = "between"

    def is_complete(self) -> bool:
        return self.state == "done" or (self.state == "number" and not self.stack and self._num_ok())

    def _num_ok(self) -> bool:
        try:
            float(self.num.decode())
            return self.num[-1:] not in (b"-", b".", b"e", b"E", b"+")
        except ValueError:
            return False

    def feed(self, c: int) -> bool:
        ch = bytes([c])
        s = self.state
        if s == "done":
            return ch in WS
        if s == "string":
            if ch == b'"':
                if self.string_is_key:
                    self.stack[-1] = "obj_colon"
                    self.state = "between"
                else:
                    self._end_value()
                return True
            if ch == b"\\":
                self.state = "escape"
                return True
            return c >= 0x20
        if s == "escape":
            if ch in b'"\\/bfnrt':
                self.state = "string"
                return True
            if ch == b"u":
                self.state, self.uni = "unicode", 0
                return True
            return False
        if s == "unicode":
            if ch in b"0123456789abcdefABCDEF":
                self.uni += 1
                if self.uni == 4:
                    self.state = "string"
                return True
            return False
        if s == "literal":
            if self.lit[self.lit_pos:self.lit_pos + 1] == ch:
                self.lit_pos += 1
                if self.lit_pos == len(self.lit):
                    self._end_value()
                return True
            return False
        if s == "number":
            if ch in b"0123456789+-.eE":
                cand = self.num + ch
                if self._num_prefix_ok(cand):
                    self.num = cand
                    return True
                return False
            if not self._num_ok():
                return False
            self._end_value()
            return self.feed(c)          # re-dispatch the delimiter
        if s == "between":
            if ch in WS:
                return True
            top = self.stack[-1] if self.stack else None
            if top == "obj_colon" and ch == b":":
                self.stack[-1] = "obj_val"
                self.state = "value"
                return True
            if top == "obj_next":
                if ch == b",":
                    self.stack[-1] = "obj_key"
                    self.state = "key"
                    return True
                if ch == b"}":
                    self.stack.pop()
                    self._end_value()
                    return True
            if top == "arr_next":
                if ch == b",":
                    self.stack[-1] = "arr_val"
                    self.state = "value"
                    return True
                if ch == b"]":
                    self.stack.pop()
                    self._end_value()
                    return True
            return False
        if s == "key":
            if ch in WS:
                return True
            if ch == b'"':
                self.state, self.string_is_key = "string", True
                return True
            if ch == b"}" and self.stack and self.stack[-1] == "obj_key_first":
                self.stack.pop()
                self._end_value()
                return True
            return False
        # value
        if ch in WS:
            return True
        if self.require_object and not self.started and ch != b"{":
            return False
        self.started = True
        if ch == b"{":
            self.stack.append("obj_key_first")
            self.state = "key"
            return True
        if ch == b"[":
            self.stack.append("arr_first")
            self.state = "value"
            return True
        if ch == b"]" and self.stack and self.stack[-1] == "arr_first":
            self.stack.pop()
            self._end_value()
            return True
        if self.stack and self.stack[-1] == "arr_first":
            self.stack[-1] = "arr_val"
        if ch == b'"':
            self.state, self.string_is_key = "string", False
            return True
        if ch in b"-0123456789":
            self.state, self.num = "number", ch
            return True
        for lit in (b"true", b"false", b"null"):
            if lit[:1] == ch:
                self.state, self.lit, self.lit_pos = "literal", lit, 1
                return True
        return False

    @staticmethod
    def _num_prefix_ok(b: bytes) -> bool:
        import re
        return re.fullmatch(rb"-?(0|[1-9]\d*)?(\.\d*)?([eE][+-]?\d*)?", b) is not None and \
            not (len(b) > 1 and b[0:1] == b"0" and b[1:2].isdigit())

    def feed_bytes(self, bs: bytes) -> bool:
        for c in bs:
            if not self.feed(c):
                return False
        return True


# obj_key_first behaves like obj_key for a quoted key
_orig_feed = JsonMatcher.feed


def _feed(self, c):
    if self.state == "key" and self.stack and self.stack[-1] == "obj_key_first" and bytes([c]) == b'"':
        self.stack[-1] = "obj_key"
    return _orig_feed(self, c)


JsonMatcher.feed = _feed


def validate_schema(value, schema: dict) -> bool:
    """JSON-schema subset check used on completed documents (type / properties / required /
    enum / items / anyOf)."""
    if not schema:
        return True
    if "anyOf" in schema:
        return any(validate_schema(value, s) for s in schema["anyOf"])
    if "enum" in schema and value not in schema["enum"]:
        return False
    t = schema.get("type")
    types = {"object": dict, "array": list, "string": str, "boolean": bool, "null": type(None)}
    if t == "integer":
        if not (isinstance(value, int) and not isinstance(value, bool)):
            return False
    elif t == "number":
        if not (isinstance(value, (int, float)) and not isinstance(value, bool)):
            return False
    elif t in types and not isinstance(value, types[t]):
        return False
    if isinstance(value, dict):
        for k in schema.get("required", []):
            if k not in value:
                return False
        for k, sub in schema.get("properties", {}).items():
            if k in value and not validate_schema(value[k], sub):
                return False
    if isinstance(value, list) and "items" in schema:
        return all(validate_schema(v, schema["items"]) for v in value)
    return True


class TokenGrammar:
    """Adapter handed to the sampler through ``SamplingParams.grammar``."""

    def __init__(self, tokenizer, matcher, eos_token_id: Optional[int] = None, probe: int = 64):
        self.tk, self.m, self.eos, self.probe = tokenizer, matcher, eos_token_id, probe
        self._last_logits: Optional[torch.Tensor] = None

    def observe_logits(self, row: torch.Tensor) -> None:
        self._last_logits = row

    def _legal(self, tid: int) -> bool:
        if tid == self.eos:
            return self.m.is_complete()
        b = self.tk.token_bytes(tid)
        if not b:
            return False
        return self.m.clone().feed_bytes(b)

    def allowed_mask(self, vocab: int) -> torch.Tensor:
        mask = torch.zeros(vocab, dtype=torch.bool)
        if self._last_logits is not None:
            order = torch.argsort(self._last_logits.float().cpu(), descending=True)
            found, width = 0, self.probe
            i = 0
            while i < vocab and (found == 0 or i < width):
                t = int(order[i])
                if self._legal(t):
                    mask[t] = True
                    found += 1
                i += 1
            if found:
                return mask
        for t in range(min(vocab, getattr(self.tk, "vocab_size", vocab))):
            if self._legal(t):
                mask[t] = True
        if not mask.any() and self.eos is not None:
            mask[self.eos] = True
        return mask

    def advance(self, tid: int) -> None:
        if tid != self.eos:
            self.m.feed_bytes(self.tk.token_bytes(tid))


def grammar_for_response_format(fmt: Optional[dict], tokenizer, eos_token_id=None) -> Optional[TokenGrammar]:
    if not fmt:
        return None
    t = fmt.get("type")
    if t in ("json_object", "json_schema"):
        from .. import native
        if native.available() and hasattr(tokenizer, "token_bytes") and hasattr(tokenizer, "vocab_size"):
            return native.NativeJsonGrammar(tokenizer, eos_token_id, require_object=True)
        return TokenGrammar(tokenizer, JsonMatcher(require_object=True), eos_token_id)
    return None
