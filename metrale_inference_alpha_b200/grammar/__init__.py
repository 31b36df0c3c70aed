"""Constrained decoding: EBNF / regular expression / JSON Schema / structural tags -> one
compiled pushdown grammar -> per-step token masks.

    g = compile_json_schema(schema)            # or compile_ebnf / compile_regex / compile_structural_tag
    m = TokenMatcher(g, tokenizer, eos_id)     # native matcher when built, Python otherwise
    mask = m.allowed_mask(vocab); m.advance(token); m.rollback(k)

Compiled grammars are immutable and cached by a hash of their source (``GrammarCache``); the
server prewarms the cache with the tool schemas of a request before its first decode step.

Role of the reference's ``crates/grammar`` (``api``, ``compiler``, ``structural_tag``, compile
cache / prewarm).
"""
from __future__ import annotations

import hashlib
import json
import threading
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence

from .ebnf import parse_ebnf
from .ir import CompiledGrammar, GrammarError, compile_rules
from .matcher import GrammarMatcher, TokenMatcher, matches
from .regex import parse_regex
from .schema import base_rules, schema_to_rules
from .structural_tag import structural_tag_rules

__all__ = ["CompiledGrammar", "GrammarError", "GrammarMatcher", "TokenMatcher", "GrammarCache", "matches",
           "compile_ebnf", "compile_regex", "compile_json_schema", "compile_json_object",
           "compile_structural_tag", "default_cache"]


class GrammarCache:
    """LRU of compiled grammars keyed by a hash of (kind, source)."""

    def __init__(self, capacity: int = 256):
        self.capacity = capacity
        self._d: "OrderedDict[str, CompiledGrammar]" = OrderedDict()
        self._lock = threading.Lock()
        self.hits = self.misses = 0

    @staticmethod
    def key(kind: str, source: str) -> str:
        return kind + ":" + hashlib.sha256(source.encode("utf-8")).hexdigest()

    def get_or_compile(self, kind: str, source: str, build) -> CompiledGrammar:
        k = self.key(kind, source)
        with self._lock:
            g = self._d.get(k)
            if g is not None:
                self._d.move_to_end(k)
                self.hits += 1
                return g
        g = build()
        g.key = k
        with self._lock:
            self.misses += 1
            self._d[k] = g
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)
        return g

    def __len__(self) -> int:
        return len(self._d)


default_cache = GrammarCache()


def compile_ebnf(text: str, root: str = "root", cache: Optional[GrammarCache] = default_cache) -> CompiledGrammar:
    build = lambda: compile_rules(parse_ebnf(text), root)
    return cache.get_or_compile("ebnf:" + root, text, build) if cache is not None else build()


def compile_regex(pattern: str, cache: Optional[GrammarCache] = default_cache) -> CompiledGrammar:
    build = lambda: compile_rules({"root": parse_regex(pattern)})
    return cache.get_or_compile("regex", pattern, build) if cache is not None else build()


def compile_json_schema(schema, cache: Optional[GrammarCache] = default_cache, max_ws: int = 8) -> CompiledGrammar:
    src = schema if isinstance(schema, str) else json.dumps(schema, sort_keys=True)
    build = lambda: compile_rules(schema_to_rules(schema, max_ws=max_ws))
    return cache.get_or_compile(f"schema:{max_ws}", src, build) if cache is not None else build()


def compile_json_object(cache: Optional[GrammarCache] = default_cache) -> CompiledGrammar:
    """Any JSON object (``response_format: json_object``)."""
    def build():
        rules = base_rules()
        rules["root"] = ("seq", [("ref", "ws"), ("ref", "object"), ("ref", "ws")])
        return compile_rules(rules)
    return cache.get_or_compile("json_object", "", build) if cache is not None else build()


def compile_structural_tag(tags: Sequence[dict], triggers: Sequence[str],
                           cache: Optional[GrammarCache] = default_cache, at_least_one: bool = False,
                           stop_after_first: bool = False, calls_only: bool = False) -> CompiledGrammar:
    """Free text in which every occurrence of a trigger must continue as one of the tags whose
    ``begin`` starts with it: ``begin`` + JSON matching ``schema`` (or the ``grammar`` rules /
    ``regex`` given instead) + ``end``. ``calls_only`` leaves no free text: the output is one or
    more tagged segments (a forced tool call)."""
    src = json.dumps({"tags": list(tags), "triggers": list(triggers), "one": at_least_one,
                      "stop": stop_after_first, "only": calls_only}, sort_keys=True, default=str)
    build = lambda: compile_rules(structural_tag_rules(tags, triggers, at_least_one, stop_after_first, calls_only))
    return cache.get_or_compile("stag", src, build) if cache is not None else build()
