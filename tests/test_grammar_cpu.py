"""Grammar engine: EBNF / regex / JSON Schema / structural-tag compilers, the pushdown matcher
(Python) and its native twin (differential), token masks, rollback, the compile cache."""
import json
import random
import re

import pytest
import torch

from metrale_inference_alpha_b200 import grammar as G
from metrale_inference_alpha_b200 import native
from metrale_inference_alpha_b200.grammar.ir import utf8_sequences


class MultiByteTokenizer:
    """256 single-byte tokens followed by multi-byte pieces (some cut UTF-8 characters)."""

    def __init__(self, extra):
        self.pieces = [bytes([i]) for i in range(256)] + [e if isinstance(e, bytes) else e.encode() for e in extra]
        self.pieces.append(b"")                 # a special token without bytes
        self.vocab_size = len(self.pieces)

    def token_bytes(self, t):
        return self.pieces[t]

    def encode_greedy(self, data: bytes):
        out, i = [], 0
        order = sorted(range(len(self.pieces) - 1), key=lambda t: -len(self.pieces[t]))
        while i < len(data):
            for t in order:
                p = self.pieces[t]
                if p and data.startswith(p, i):
                    out.append(t)
                    i += len(p)
                    break
        return out


EXTRA = ['{"', '":', '", "', '"}', "name", "age", "true", "false", "null", " ", "  ", "\n", "12", "3.5", "e+", '"name"',
         '"name": "', "<tool_call>", "</tool_call>", "<tool", "_call>", "abc", "é", "é".encode()[:1], "日本".encode(),
         "日本".encode()[:4], '{"name": "f", "arguments": ', "}\n", "[", "]", ", ", "[]", "{}", '""', "\\n", '\\"']


def test_utf8_sequences_cover_exactly():
    rnd = random.Random(0)
    for lo, hi in [(0x80, 0x7FF), (0x7FF, 0x800), (0xD000, 0xE100), (0xFFFF, 0x10000), (0x80, 0x10FFFF), (0x3042, 0x3093)]:
        seqs = utf8_sequences(lo, hi)

        def accepts(bs):
            return any(len(bs) == len(s) and all(a <= c <= b for c, (a, b) in zip(bs, s)) for s in seqs)
        for cp in [lo, hi, (lo + hi) // 2] + [rnd.randint(lo, hi) for _ in range(200)]:
            if 0xD800 <= cp <= 0xDFFF:
                continue
            assert accepts(chr(cp).encode()), hex(cp)
        for cp in [lo - 1, hi + 1]:
            if 0 <= cp <= 0x10FFFF and not 0xD800 <= cp <= 0xDFFF:
                assert not accepts(chr(cp).encode()), hex(cp)


def test_ebnf_basic_and_errors():
    g = G.compile_ebnf('''
        root ::= "{" ws pair ("," ws pair)* "}"   # an object of lower-case keys
        pair ::= str ":" ws num
        str  ::= "\\"" [a-z]+ "\\""
        num  ::= [0-9]{1,3}
        ws   ::= " "?
    ''', cache=None)
    assert G.matches(g, b'{"ab": 12, "c":7}')
    assert not G.matches(g, b'{"ab": 1234}')
    assert not G.matches(g, b"{}")
    with pytest.raises(G.GrammarError):
        G.compile_ebnf('root ::= root "a" | "b"', cache=None)           # left recursion
    with pytest.raises(G.GrammarError):
        G.compile_ebnf('root ::= missing', cache=None)
    with pytest.raises(G.GrammarError):
        G.compile_ebnf('root ::= "a" root ::= "b"', cache=None)
    # right recursion, nested groups, negated class, unicode escape, any-char
    g2 = G.compile_ebnf('root ::= item ("," root)?\nitem ::= [^,\\x00-\\x1f]+ | "\\u00e9" .', cache=None)
    assert G.matches(g2, "a,b,c".encode()) and G.matches(g2, "é日,x".encode()) and not G.matches(g2, b"a,,b")


@pytest.mark.parametrize("pat,good,bad", [
    (r"(\d{3})-[a-c]+(?:x|yz)?", ["123-abc", "000-ayz"], ["12-a", "123-", "123-ad"]),
    (r"[A-Z][a-z]*( [A-Z][a-z]*)*", ["Hello World", "A"], ["hello", "Hello  World"]),
    (r"\w+@\w+\.(com|org)", ["a_b@c.com"], ["a@b.net", "@b.com"]),
    (r"^-?(0|[1-9]\d*)(\.\d+)?$", ["0", "-12.50", "7"], ["01", "1.", "--1"]),
    (r"[^\s\d]{2,4}é+", ["abé", "日本語éé"], ["a1é", "abcdeé", "ab"]),
    (r"a{2}b{1,}c{0,2}", ["aab", "aabbbcc"], ["ab", "aabccc"]),
    (r"(?P<y>\d{4})-(?<m>\d\d)", ["2024-05"], ["2024-5"]),
])
def test_regex_against_python_re(pat, good, bad):
    g = G.compile_regex(pat, cache=None)
    for s in good:
        assert re.fullmatch(pat.replace("(?<m>", "(?P<m>"), s), s
        assert G.matches(g, s.encode()), (pat, s)
    for s in bad:
        assert not G.matches(g, s.encode()), (pat, s)


def test_regex_refuses_what_it_cannot_express():
    for pat in [r"(a)\1", r"(?=a)b", r"a\b", r"\p{L}+", r"*a"]:
        with pytest.raises(G.GrammarError):
            G.compile_regex(pat, cache=None)


SCHEMA = {
    "type": "object",
    "properties": {
        "name": {"type": "string", "minLength": 1},
        "age": {"type": "integer", "minimum": 0},
        "tags": {"type": "array", "items": {"type": "string"}, "minItems": 1, "maxItems": 3},
        "kind": {"enum": ["a", "b", 3, None]},
        "pos": {"type": "array", "prefixItems": [{"type": "number"}, {"type": "number"}], "items": False},
        "when": {"type": "string", "format": "date"},
        "id": {"type": "string", "pattern": "^[A-Z]{2}\\d{2}$"},
        "opt": {"type": ["string", "null"]},
        "inner": {"$ref": "#/$defs/inner"},
    },
    "required": ["name", "age"],
    "$defs": {"inner": {"type": "object", "properties": {"x": {"type": "boolean"}}, "required": ["x"],
                        "additionalProperties": {"type": "integer"}}},
}


def test_json_schema_accepts_and_refuses():
    g = G.compile_json_schema(SCHEMA, cache=None)
    good = [
        {"name": "x", "age": 3},
        {"name": "x", "age": 0, "tags": ["a", "b"], "kind": "a"},
        {"name": "é\n\"q\"", "age": 12, "kind": None, "pos": [1.5, -2e3], "when": "2024-02-29", "id": "AB12", "opt": None},
        {"name": "x", "age": 1, "inner": {"x": True, "k": 4, "j": -1}},
    ]
    for v in good:
        for text in (json.dumps(v), json.dumps(v, separators=(",", ":")), json.dumps(v, indent=1, ensure_ascii=False)):
            assert G.matches(g, text.encode()), text
    bad = [
        '{"age":3}', '{"name":"x","age":-3}', '{"name":"","age":3}', '{"name":"x","age":3,"tags":[]}',
        '{"name":"x","age":3,"tags":["a","b","c","d"]}', '{"name":"x","age":3,"other":1}', '{"name":"x","age":3,"kind":"c"}',
        '{"age":3,"name":"x"}', '{"name":"x","age":3,"pos":[1]}', '{"name":"x","age":3,"pos":[1,2,3]}',
        '{"name":"x","age":3,"when":"2024-13-01"}', '{"name":"x","age":3,"id":"ab12"}', '{"name":"x","age":3.5}',
        '{"name":"x","age":3,"inner":{"k":4}}', '{"name":"x","age":3,"inner":{"x":true,"k":"s"}}', '{"name":"x","age":3,}',
    ]
    for text in bad:
        assert not G.matches(g, text.encode()), text


def test_json_schema_recursive_anyof_allof_const():
    rec = {"$defs": {"node": {"type": "object", "properties": {"v": {"type": "number"},
                                                                 "kids": {"type": "array", "items": {"$ref": "#/$defs/node"}}},
                              "required": ["v"]}}, "$ref": "#/$defs/node"}
    g = G.compile_json_schema(rec, cache=None)
    assert G.matches(g, b'{"v":1.5e3,"kids":[{"v":2},{"v":3,"kids":[]}]}')
    assert not G.matches(g, b'{"kids":[]}')
    g = G.compile_json_schema({"anyOf": [{"type": "integer"}, {"const": "none"}, {"type": "array", "items": {"type": "boolean"}}]},
                              cache=None)
    assert all(G.matches(g, t) for t in (b"12", b'"none"', b"[true, false]", b"[]"))
    assert not any(G.matches(g, t) for t in (b'"x"', b"1.5", b"[1]"))
    g = G.compile_json_schema({"allOf": [{"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]},
                                         {"type": "object", "properties": {"b": {"type": "string"}}, "required": ["b"]}]},
                              cache=None)
    assert G.matches(g, b'{"a":1,"b":"x"}') and not G.matches(g, b'{"a":1}')
    assert G.matches(G.compile_json_schema(True, cache=None), b'[1, {"a": null}]')
    assert G.matches(G.compile_json_object(cache=None), b' {"a":[1,2,{"b":null}]} ')
    assert not G.matches(G.compile_json_object(cache=None), b"[1]")


TAGS = [{"begin": '<tool_call>\n{"name": "f", "arguments": ',
         "schema": {"type": "object", "properties": {"x": {"type": "integer"}}, "required": ["x"]},
         "end": "}\n</tool_call>"},
        {"begin": '<tool_call>\n{"name": "g", "arguments": ', "schema": {"type": "object"}, "end": "}\n</tool_call>"}]


def test_structural_tag_free_text_and_constrained_segments():
    g = G.compile_structural_tag(TAGS, ["<tool_call>"], cache=None)
    ok = 'hello <tool <<tool_call>\n{"name": "f", "arguments": {"x": 5}}\n</tool_call> bye é <tool_call>\n{"name": "g", "arguments": {"k": [1]}}\n</tool_call>'
    assert G.matches(g, ok.encode())
    assert G.matches(g, b"just text") and G.matches(g, b"")
    assert not G.matches(g, b'text <tool_call>{"x":5}')
    assert not G.matches(g, b'<tool_call>\n{"name": "f", "arguments": {"y": 5}}\n</tool_call>')
    assert not G.matches(g, b'<tool_call>\n{"name": "h", "arguments": {}}\n</tool_call>')
    m = G.GrammarMatcher(g)
    assert m.feed_bytes(b"a" * 4000) and len(m.frames) == 0          # tail calls: no stack growth in free text
    one = G.compile_structural_tag(TAGS, ["<tool_call>"], cache=None, at_least_one=True, stop_after_first=True)
    assert not G.matches(one, b"just text")
    assert G.matches(one, b'x<tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call>')
    assert not G.matches(one, b'x<tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call> more')
    with pytest.raises(G.GrammarError):
        G.compile_structural_tag([{"begin": "<x>", "schema": True, "end": ""}], ["<tool_call>"], cache=None)


def _walk(tm, tk, data: bytes):
    """Feeds `data` token by token, checking every token against the mask first."""
    for t in tk.encode_greedy(data):
        mask = tm.allowed_mask(tk.vocab_size)
        assert bool(mask[t]), (t, tk.token_bytes(t))
        tm.advance(t)


def test_token_mask_python_matcher():
    tk = MultiByteTokenizer(EXTRA)
    eos = tk.vocab_size - 1
    tm = G.TokenMatcher(G.compile_json_schema(SCHEMA, cache=None), tk, eos, prefer_native=False)
    mask = tm.allowed_mask(tk.vocab_size)
    legal = {tk.token_bytes(t) for t in torch.nonzero(mask).flatten().tolist()}
    assert b"{" in legal and b'{"' in legal and b" " in legal and b"[" not in legal and b"a" not in legal
    assert not mask[eos]
    _walk(tm, tk, b'{"name": "ab\xc3\xa9", "age": 12}')
    assert tm.is_complete() and tm.allowed_mask(tk.vocab_size)[eos]
    tm.rollback(2)
    assert not tm.is_complete()


@pytest.mark.skipif(not (native.available() and native.has_pda()), reason="native runtime not built")
def test_native_matcher_equals_python_on_masks_and_rollback():
    tk = MultiByteTokenizer(EXTRA)
    eos = tk.vocab_size - 1
    cases = [
        (G.compile_json_schema(SCHEMA, cache=None),
         json.dumps({"name": "日本 é", "age": 12, "tags": ["abc", ""], "kind": 3, "pos": [3.5, 1e+2], "opt": None,
                     "inner": {"x": False, "k": 12}}, ensure_ascii=False).encode()),
        (G.compile_structural_tag(TAGS, ["<tool_call>"], cache=None),
         'é <tool <tool_call>\n{"name": "f", "arguments": {"x": 12}}\n</tool_call> abc 日本'.encode()),
        (G.compile_regex(r"(abc|é|\d{2,3}| )+\.", cache=None), "abc 12 é 123.".encode()),
        (G.compile_ebnf('root ::= "[" (v ("," v)*)? "]"\nv ::= [0-9]+ | root', cache=None), b"[12,[3,[],[12]],12]"),
    ]
    for g, data in cases:
        a = G.TokenMatcher(g, tk, eos, prefer_native=True)
        b = G.TokenMatcher(g, tk, eos, prefer_native=False)
        assert a._native is not None and b._py is not None
        toks = tk.encode_greedy(data)
        for i, t in enumerate(toks):
            ma, mb = a.allowed_mask(tk.vocab_size), b.allowed_mask(tk.vocab_size)
            assert torch.equal(ma, mb), (i, torch.nonzero(ma != mb).flatten().tolist())
            assert bool(ma[t])
            a.advance(t)
            b.advance(t)
            if i % 5 == 4:                       # speculative rewind: drop two tokens, replay them
                a.rollback(2)
                b.rollback(2)
                assert torch.equal(a.allowed_mask(tk.vocab_size), b.allowed_mask(tk.vocab_size))
                for r in toks[i - 1:i + 1]:
                    a.advance(r)
                    b.advance(r)
        assert a.is_complete() and b.is_complete()
        assert torch.equal(a.allowed_mask(tk.vocab_size), b.allowed_mask(tk.vocab_size))
        st = a._native.stats()
        assert st["mask_cache_hits"] > 0


@pytest.mark.skipif(not (native.available() and native.has_pda()), reason="native runtime not built")
def test_native_matcher_pickles_by_replay():
    import pickle
    tk = MultiByteTokenizer(EXTRA)
    tm = G.TokenMatcher(G.compile_json_object(cache=None), tk, tk.vocab_size - 1)
    for t in tk.encode_greedy(b'{"name": [12'):
        tm.advance(t)
    tm2 = pickle.loads(pickle.dumps(tm))
    assert torch.equal(tm.allowed_mask(tk.vocab_size), tm2.allowed_mask(tk.vocab_size))


def test_compile_cache_hits_and_evicts():
    c = G.GrammarCache(capacity=2)
    a = G.compile_regex("a+", cache=c)
    assert G.compile_regex("a+", cache=c) is a and c.hits == 1 and c.misses == 1
    G.compile_regex("b+", cache=c)
    G.compile_regex("c+", cache=c)
    assert len(c) == 2
    assert G.compile_regex("a+", cache=c) is not a            # evicted, recompiled
