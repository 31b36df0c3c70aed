"""JSON Schema -> grammar IR.

Covers what tool definitions and ``response_format: json_schema`` use in practice: ``type``
(also as a list), ``enum``, ``const``, ``properties`` / ``required`` / ``additionalProperties``,
``items`` / ``prefixItems`` / ``minItems`` / ``maxItems``, ``anyOf`` / ``oneOf``, single-branch or
object-merging ``allOf``, ``$ref`` into ``$defs`` / ``definitions`` (recursive schemas become
recursive rules), strings with ``pattern`` / ``minLength`` / ``maxLength`` / ``format`` (date,
time, date-time, uuid, email, ipv4), integers and numbers (bounds that fit a sign are enforced:
``minimum >= 0`` forbids the minus sign). Properties are emitted in declaration order, required
ones always, optional ones skippable. Keywords that do not restrict the syntax (``title``,
``description``, ``default``, ``examples``) are ignored; an empty or ``true`` schema is any JSON.

Role of the reference's ``crates/grammar/src/schema``.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

from .ir import GrammarError
from .regex import parse_regex

WS = ("ref", "ws")


def _lit(s: str) -> tuple:
    return ("lit", s.encode("utf-8"))


def base_rules(max_ws: int = 8) -> Dict[str, tuple]:
    """The JSON core every schema grammar shares."""
    digit = ("cls", [(48, 57)], False)
    hexd = ("cls", [(48, 57), (65, 70), (97, 102)], False)
    integer = ("seq", [("rep", _lit("-"), 0, 1),
                       ("alt", [_lit("0"), ("seq", [("cls", [(49, 57)], False), ("rep", digit, 0, None)])])])
    number = ("seq", [("ref", "integer"),
                      ("rep", ("seq", [_lit("."), ("rep", digit, 1, None)]), 0, 1),
                      ("rep", ("seq", [("cls", [(69, 69), (101, 101)], False),
                                       ("rep", ("cls", [(43, 43), (45, 45)], False), 0, 1),
                                       ("rep", digit, 1, None)]), 0, 1)])
    char = ("alt", [("cls", [(0, 0x1F), (34, 34), (92, 92)], True),
                    ("seq", [_lit("\\"), ("alt", [("cls", [(c, c) for c in b'"\\/bfnrt'], False),
                                                   ("seq", [_lit("u"), ("rep", hexd, 4, 4)])])])])
    return {
        "ws": ("rep", ("cls", [(9, 10), (13, 13), (32, 32)], False), 0, max_ws),
        "integer": integer,
        "number": number,
        "char": char,
        "string": ("seq", [_lit('"'), ("rep", ("ref", "char"), 0, None), _lit('"')]),
        "boolean": ("alt", [_lit("true"), _lit("false")]),
        "null": _lit("null"),
        "value": ("alt", [("ref", "object"), ("ref", "array"), ("ref", "string"), ("ref", "number"),
                          ("ref", "boolean"), ("ref", "null")]),
        "member": ("seq", [("ref", "string"), WS, _lit(":"), WS, ("ref", "value")]),
        "object": ("seq", [_lit("{"), WS,
                           ("rep", ("seq", [("ref", "member"),
                                            ("rep", ("seq", [WS, _lit(","), WS, ("ref", "member")]), 0, None), WS]), 0, 1),
                           _lit("}")]),
        "array": ("seq", [_lit("["), WS,
                          ("rep", ("seq", [("ref", "value"),
                                           ("rep", ("seq", [WS, _lit(","), WS, ("ref", "value")]), 0, None), WS]), 0, 1),
                          _lit("]")]),
    }


_FORMATS = {
    "date": r"\d{4}-(0[1-9]|1[0-2])-(0[1-9]|[12]\d|3[01])",
    "time": r"([01]\d|2[0-3]):[0-5]\d:[0-5]\d(\.\d+)?(Z|[+-]([01]\d|2[0-3]):[0-5]\d)?",
    "date-time": r"\d{4}-(0[1-9]|1[0-2])-(0[1-9]|[12]\d|3[01])T([01]\d|2[0-3]):[0-5]\d:[0-5]\d(\.\d+)?(Z|[+-]([01]\d|2[0-3]):[0-5]\d)",
    "uuid": r"[0-9a-fA-F]{8}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{12}",
    "email": r"[A-Za-z0-9._%+-]+@[A-Za-z0-9-]+(\.[A-Za-z0-9-]+)+",
    "ipv4": r"((25[0-5]|2[0-4]\d|1?\d?\d)\.){3}(25[0-5]|2[0-4]\d|1?\d?\d)",
}


class _Conv:
    def __init__(self, root_schema, max_ws: int):
        self.root = root_schema
        self.rules = base_rules(max_ws)
        self.ref_rule: Dict[str, str] = {}
        self.n = 0

    def fresh(self, hint: str) -> str:
        self.n += 1
        return f"{hint}_{self.n}"

    def define(self, hint: str, body: tuple) -> tuple:
        name = self.fresh(hint)
        self.rules[name] = body
        return ("ref", name)

    def resolve(self, ref: str):
        if not ref.startswith("#"):
            raise GrammarError(f"only local $ref is supported: {ref}")
        node = self.root
        for part in ref[1:].split("/"):
            if not part:
                continue
            part = part.replace("~1", "/").replace("~0", "~")
            if isinstance(node, list):
                node = node[int(part)]
            elif isinstance(node, dict) and part in node:
                node = node[part]
            else:
                raise GrammarError(f"unresolvable $ref {ref}")
        return node

    # ------------------------------------------------------------------ per type
    def string(self, s: dict) -> tuple:
        if "pattern" in s:
            pat = s["pattern"]
            body = parse_regex(pat)
            return ("seq", [_lit('"'), self.define("pattern", body), _lit('"')])
        if s.get("format") in _FORMATS:
            return ("seq", [_lit('"'), self.define("format", parse_regex(_FORMATS[s["format"]])), _lit('"')])
        lo, hi = int(s.get("minLength", 0)), s.get("maxLength")
        if lo == 0 and hi is None:
            return ("ref", "string")
        if hi is not None and int(hi) > 4096:
            hi = None
        return ("seq", [_lit('"'), ("rep", ("ref", "char"), lo, None if hi is None else int(hi)), _lit('"')])

    def number(self, s: dict, integer: bool) -> tuple:
        lo = s.get("minimum", s.get("exclusiveMinimum"))
        hi = s.get("maximum", s.get("exclusiveMaximum"))
        base = "integer" if integer else "number"
        if lo is not None and lo >= 0:
            # non-negative: drop the sign
            digit = ("cls", [(48, 57)], False)
            nat = ("alt", [_lit("0"), ("seq", [("cls", [(49, 57)], False), ("rep", digit, 0, None)])])
            if integer:
                return nat
            tail = self.rules["number"][1][1:]
            return ("seq", [nat] + list(tail))
        if hi is not None and hi < 0:
            digit = ("cls", [(48, 57)], False)
            neg = ("seq", [_lit("-"), ("alt", [_lit("0"), ("seq", [("cls", [(49, 57)], False), ("rep", digit, 0, None)])])])
            if integer:
                return neg
            tail = self.rules["number"][1][1:]
            return ("seq", [neg] + list(tail))
        return ("ref", base)

    def array(self, s: dict) -> tuple:
        prefix = s.get("prefixItems") or (s["items"] if isinstance(s.get("items"), list) else [])
        items = s.get("items") if not isinstance(s.get("items"), list) else s.get("additionalItems", True)
        lo = int(s.get("minItems", 0))
        hi = s.get("maxItems")
        sep = ("seq", [WS, _lit(","), WS])
        parts: List[tuple] = [self.convert(p) for p in prefix]
        if items is False:
            rest_lo, rest_hi, item = 0, 0, None
        else:
            item = self.convert(items if isinstance(items, dict) else True)
            rest_lo = max(0, lo - len(parts))
            rest_hi = None if hi is None else max(0, int(hi) - len(parts))
        body: List[tuple] = []
        if parts:
            seq = [parts[0]]
            for p in parts[1:]:
                seq += [sep, p]
            if item is not None and (rest_hi is None or rest_hi > 0):
                seq.append(("rep", ("seq", [sep, item]), rest_lo, rest_hi))
            body = seq
            inner = ("seq", body + [WS])
        elif item is None:
            inner = ("empty",)
        else:
            if rest_hi == 0:
                inner = ("empty",)
            else:
                more = ("rep", ("seq", [sep, item]), max(0, rest_lo - 1), None if rest_hi is None else rest_hi - 1)
                one = ("seq", [item, more, WS])
                inner = one if rest_lo > 0 else ("rep", one, 0, 1)
        return ("seq", [_lit("["), WS, inner, _lit("]")])

    def obj(self, s: dict) -> tuple:
        props: Dict[str, object] = s.get("properties") or {}
        required = set(s.get("required") or [])
        addl = s.get("additionalProperties", True if not props else False)
        if not props and addl is True and not required:
            return ("ref", "object")
        sep = ("seq", [WS, _lit(","), WS])

        def member(key: str, sub) -> tuple:
            return ("seq", [_lit(json.dumps(key, ensure_ascii=False)), WS, _lit(":"), WS, self.convert(sub)])
        names = list(props.keys())
        for r in required:
            if r not in props:
                names.append(r)
        mems = [(k, member(k, props.get(k, True)), k in required) for k in names]
        extra = None
        if addl is not False:
            sub = self.convert(addl if isinstance(addl, dict) else True)
            extra = ("seq", [("ref", "string"), WS, _lit(":"), WS, sub])
        # tail(i, started): members i.. given whether one was already written. Built back to
        # front as rules so that shared suffixes are not duplicated.
        n = len(mems)
        tail_started: List[Optional[tuple]] = [None] * (n + 1)
        tail_fresh: List[Optional[tuple]] = [None] * (n + 1)
        tail_started[n] = ("rep", ("seq", [sep, extra]), 0, None) if extra is not None else ("empty",)
        if extra is not None:
            tail_fresh[n] = ("rep", ("seq", [extra, ("rep", ("seq", [sep, extra]), 0, None)]), 0, 1)
        else:
            tail_fresh[n] = ("empty",)
        for i in range(n - 1, -1, -1):
            _, m, req = mems[i]
            with_s = ("seq", [sep, m, tail_started[i + 1]])
            with_f = ("seq", [m, tail_started[i + 1]])
            if req:
                ts, tf = with_s, with_f
            else:
                ts, tf = ("alt", [with_s, tail_started[i + 1]]), ("alt", [with_f, tail_fresh[i + 1]])
            tail_started[i] = self.define("obj_s", ts)
            tail_fresh[i] = self.define("obj_f", tf)
        return ("seq", [_lit("{"), WS, tail_fresh[0], WS, _lit("}")])

    # ------------------------------------------------------------------ dispatch
    def convert(self, s) -> tuple:
        if s is True or s == {} or s is None:
            return ("ref", "value")
        if s is False:
            return ("cls", [], False)
        if not isinstance(s, dict):
            raise GrammarError("schema must be an object or a boolean")
        if "$ref" in s:
            ref = s["$ref"]
            if ref not in self.ref_rule:
                name = self.fresh("ref")
                self.ref_rule[ref] = name
                self.rules[name] = ("empty",)             # placeholder: breaks recursion
                self.rules[name] = self.convert(self.resolve(ref))
            return ("ref", self.ref_rule[ref])
        if "const" in s:
            return _lit(json.dumps(s["const"], ensure_ascii=False, separators=(",", ":")))
        if "enum" in s:
            return ("alt", [_lit(json.dumps(v, ensure_ascii=False, separators=(",", ":"))) for v in s["enum"]])
        for k in ("anyOf", "oneOf"):
            if k in s:
                return self.define(k.lower(), ("alt", [self.convert(x) for x in s[k]]))
        if "allOf" in s:
            subs = s["allOf"]
            if len(subs) == 1:
                return self.convert(subs[0])
            merged: dict = {"type": "object", "properties": {}, "required": []}
            for x in subs:
                if "$ref" in x:
                    x = self.resolve(x["$ref"])
                if x.get("type", "object") != "object":
                    raise GrammarError("allOf is supported for object schemas only")
                merged["properties"].update(x.get("properties") or {})
                merged["required"] += list(x.get("required") or [])
                if "additionalProperties" in x:
                    merged["additionalProperties"] = x["additionalProperties"]
            return self.convert(merged)
        t = s.get("type")
        if isinstance(t, list):
            return ("alt", [self.convert({**s, "type": x}) for x in t])
        if t is None:
            if "properties" in s or "required" in s:
                t = "object"
            elif "items" in s or "prefixItems" in s:
                t = "array"
            else:
                return ("ref", "value")
        if s.get("nullable") is True and t != "null":
            return ("alt", [self.convert({k: v for k, v in s.items() if k != "nullable"}), ("ref", "null")])
        if t == "string":
            return self.string(s)
        if t == "integer":
            return self.number(s, True)
        if t == "number":
            return self.number(s, False)
        if t == "boolean":
            return ("ref", "boolean")
        if t == "null":
            return ("ref", "null")
        if t == "array":
            return self.define("array", self.array(s))
        if t == "object":
            return self.define("object", self.obj(s))
        raise GrammarError(f"unsupported schema type {t!r}")


def schema_to_rules(schema, root: str = "root", max_ws: int = 8) -> Dict[str, tuple]:
    if isinstance(schema, (str, bytes)):
        schema = json.loads(schema)
    c = _Conv(schema, max_ws)
    body = c.convert(schema)
    c.rules[root] = ("seq", [WS, body, WS])
    return c.rules
