"""Constrained decoding: an incremental matcher decides which tokens may come next.

The general engine is the ``grammar`` package (EBNF / regex / JSON Schema / structural tags ->
pushdown matcher, native mask fill); this module is the server-side glue that maps request fields
to it, plus ``JsonMatcher``, the stand-alone JSON recogniser used when the native runtime is not
built. ``TokenGrammar`` lifts a byte matcher to the token vocabulary: the
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
        self._snaps: list = []              # matcher before each accepted token (speculative rewind)

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
            self._snaps.append(self.m.clone())
            self.m.feed_bytes(self.tk.token_bytes(tid))

    def rollback(self, n: int) -> None:
        for _ in range(min(n, len(self._snaps))):
            self.m = self._snaps.pop()


def _native_ok(tokenizer) -> bool:
    return hasattr(tokenizer, "token_bytes") and hasattr(tokenizer, "vocab_size")


def grammar_for_response_format(fmt: Optional[dict], tokenizer, eos_token_id=None):
    """``response_format`` -> a token matcher (None = unconstrained). ``json_object`` is any JSON
    object; ``json_schema`` is compiled by the grammar package (``json_schema.schema`` or a
    top-level ``schema``); ``regex`` (``pattern``) and ``grammar`` / ``ebnf`` (``grammar``) are
    extensions that reach the same engine. A source that does not compile raises GrammarError."""
    if not fmt:
        return None
    from .. import grammar as G
    t = fmt.get("type")
    if t == "json_schema":
        js = fmt.get("json_schema") or {}
        schema = js.get("schema", fmt.get("schema"))
        if schema is not None and _native_ok(tokenizer):
            return G.TokenMatcher(G.compile_json_schema(schema), tokenizer, eos_token_id)
        t = "json_object"
    if t == "json_object":
        from .. import native
        if native.available() and _native_ok(tokenizer):
            return native.NativeJsonGrammar(tokenizer, eos_token_id, require_object=True)
        return TokenGrammar(tokenizer, JsonMatcher(require_object=True), eos_token_id)
    if t == "regex" and _native_ok(tokenizer):
        return G.TokenMatcher(G.compile_regex(fmt.get("pattern") or fmt.get("regex") or ""), tokenizer, eos_token_id)
    if t in ("grammar", "ebnf") and _native_ok(tokenizer):
        return G.TokenMatcher(G.compile_ebnf(fmt.get("grammar") or fmt.get("ebnf") or ""), tokenizer, eos_token_id)
    return None


def response_format_from_guided(body: dict) -> Optional[dict]:
    """vLLM-style request fields (`guided_json`, `guided_regex`, `guided_grammar`, `guided_choice`, or
    the same keys inside `structured_outputs`) as an equivalent `response_format`."""
    so = body.get("structured_outputs") if isinstance(body.get("structured_outputs"), dict) else {}
    pick = lambda k: body.get("guided_" + k) if body.get("guided_" + k) is not None else so.get(k)
    js = pick("json")
    if js is not None:
        return {"type": "json_schema", "json_schema": {"schema": json.loads(js) if isinstance(js, str) else js}}
    if pick("regex"):
        return {"type": "regex", "pattern": pick("regex")}
    if pick("grammar"):
        return {"type": "ebnf", "grammar": pick("grammar")}
    choice = pick("choice")
    if choice:
        alts = " | ".join(json.dumps(str(c)) for c in choice)      # JSON string quoting is valid EBNF literal quoting
        return {"type": "ebnf", "grammar": f"root ::= {alts}"}
    return None


def tool_call_grammar(tools: Optional[List[dict]], parser: str, mode: str = "auto"):
    """Compiled grammar that keeps tool calls well-formed for the call syntax `parser` scans
    (reference: ``GrammarSpec::ToolCall``, compiled by the parser that reads the response).
    `mode`: "auto" = free text where a trigger must continue as a valid call; "required" = nothing
    but calls (the forced tool call of ``tool_choice: required`` or a named function). None when the format has no grammar here (the parser's salvage passes still
    apply)."""
    if not tools:
        return None
    from .. import grammar as G
    fns = []
    for t in tools:
        f = t.get("function") or t
        if f.get("name"):
            fns.append((f["name"], f.get("parameters") or f.get("input_schema") or {"type": "object"}))
    if not fns:
        return None
    required = mode == "required"
    if parser in ("hermes", "qwen3", "qwen"):
        tags = [{"begin": '<tool_call>\n{"name": ' + json.dumps(n) + ', "arguments": ', "schema": p,
                 "end": "}\n</tool_call>"} for n, p in fns]
        return G.compile_structural_tag(tags, ["<tool_call>"], calls_only=required)
    call = {"anyOf": [{"type": "object", "properties": {"name": {"const": n}, "arguments": p},
                       "required": ["name", "arguments"]} for n, p in fns]}
    if parser == "mistral":
        tags = [{"begin": "[TOOL_CALLS]", "schema": {"type": "array", "items": call, "minItems": 1}, "end": ""}]
        return G.compile_structural_tag(tags, ["[TOOL_CALLS]"], calls_only=required, stop_after_first=required)
    if parser == "bare_json" and required:
        return G.compile_json_schema(call)
    return None


def prewarm(tools: Optional[List[dict]], parser: str) -> int:
    """Compiles (into the shared cache) the grammars a request with these tools may need, so that
    the first constrained step does not pay for it. Returns how many compiled."""
    n = 0
    for mode in ("auto", "required"):
        try:
            n += tool_call_grammar(tools, parser, mode) is not None
        except ValueError:
            pass
    return n
