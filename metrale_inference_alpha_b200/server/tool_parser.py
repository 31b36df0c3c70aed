"""Tool-call extraction from generated text. Formats: hermes (``<tool_call>{json}</tool_call>``),
qwen3_xml (``<tool_call><function=name><parameter=k>v</parameter></function></tool_call>``),
mistral (``[TOOL_CALLS][{...}]``), bare_json (an un-enveloped ``{"name":..,"arguments":..}``).
An ordered primary / salvage pipeline, fuzzy tool-name matching and argument type coercion
against the declared schema; text before the first ``</think>`` is never parsed for calls.
Role of ``crates/server/src/tool_parser/`` (``pipeline.rs``, ``parse_dispatch.rs``)."""
from __future__ import annotations

import difflib
import json
import re
import uuid
from typing import Any, Dict, List, Optional, Tuple


def _call(name: str, args: Any) -> Dict[str, Any]:
    if not isinstance(args, str):
        args = json.dumps(args, ensure_ascii=False)
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function", "function": {"name": name, "arguments": args}}


def _json_objects(text: str):
    """Yield (start, end, obj) for every balanced top-level JSON object in text."""
    dec = json.JSONDecoder()
    i = 0
    while True:
        i = text.find("{", i)
        if i < 0:
            return
        try:
            obj, end = dec.raw_decode(text, i)
            yield i, end, obj
            i = end
        except json.JSONDecodeError:
            i += 1


def parse_hermes(text: str) -> Tuple[str, List[dict]]:
    calls, keep, pos = [], [], 0
    for m in re.finditer(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", text, re.S):
        keep.append(text[pos:m.start()])
        pos = m.end()
        try:
            o = json.loads(m.group(1))
            calls.append(_call(o["name"], o.get("arguments", o.get("parameters", {}))))
        except Exception:
            keep.append(m.group(0))
    keep.append(text[pos:])
    return "".join(keep).strip(), calls


def parse_qwen3_xml(text: str) -> Tuple[str, List[dict]]:
    calls, keep, pos = [], [], 0
    for m in re.finditer(r"<tool_call>\s*<function=([^>\s]+)>(.*?)</function>\s*(?:</tool_call>)?", text, re.S):
        keep.append(text[pos:m.start()])
        pos = m.end()
        args = {k: v.strip("\n") for k, v in re.findall(r"<parameter=([^>\s]+)>(.*?)</parameter>", m.group(2), re.S)}
        calls.append(_call(m.group(1), args))
    keep.append(text[pos:])
    return "".join(keep).strip(), calls


def parse_mistral(text: str) -> Tuple[str, List[dict]]:
    i = text.find("[TOOL_CALLS]")
    if i < 0:
        return text, []
    try:
        arr = json.loads(text[i + len("[TOOL_CALLS]"):].strip())
        arr = arr if isinstance(arr, list) else [arr]
        return text[:i].strip(), [_call(o["name"], o.get("arguments", {})) for o in arr]
    except Exception:
        return text, []


def parse_bare_json(text: str) -> Tuple[str, List[dict]]:
    calls, spans = [], []
    for s, e, o in _json_objects(text):
        if isinstance(o, dict) and isinstance(o.get("name"), str) and ("arguments" in o or "parameters" in o):
            calls.append(_call(o["name"], o.get("arguments", o.get("parameters"))))
            spans.append((s, e))
    for s, e in reversed(spans):
        text = text[:s] + text[e:]
    return text.strip(), calls


def _loose_value(v: str):
    """A parameter body: JSON when it parses, else the raw text."""
    v = v.strip()
    try:
        return json.loads(v)
    except Exception:
        return v


def parse_minimax_xml(text: str) -> Tuple[str, List[dict]]:
    """``<minimax:tool_call><invoke name="f"><parameter name="k">v</parameter></invoke></minimax:tool_call>``"""
    calls, keep, pos = [], [], 0
    for m in re.finditer(r"<minimax:tool_call>(.*?)(?:</minimax:tool_call>|$)", text, re.S):
        found = False
        for inv in re.finditer(r'<invoke name="([^"]+)">(.*?)</invoke>', m.group(1), re.S):
            args = {k: v.strip("\n") for k, v in re.findall(r'<parameter name="([^"]+)">(.*?)</parameter>', inv.group(2), re.S)}
            calls.append(_call(inv.group(1), args))
            found = True
        if found:
            keep.append(text[pos:m.start()])
            pos = m.end()
    keep.append(text[pos:])
    return "".join(keep).strip(), calls


def parse_gemma4(text: str) -> Tuple[str, List[dict]]:
    """``<|tool_call>call:fn_name{key:val,...}<tool_call|>``; values are JSON scalars / strings,
    bare words are taken as strings."""
    calls, keep, pos = [], [], 0
    for m in re.finditer(r"<\|tool_call>\s*call:([\w.\-]+)\s*\{(.*?)\}\s*<tool_call\|>", text, re.S):
        body, args, ok = m.group(2), {}, True
        depth, cur, parts, in_str = 0, "", [], False
        for ch in body:                                   # split on top-level commas
            if ch == '"' and not cur.endswith("\\"):
                in_str = not in_str
            if not in_str:
                if ch in "[{":
                    depth += 1
                elif ch in "]}":
                    depth -= 1
                elif ch == "," and depth == 0:
                    parts.append(cur)
                    cur = ""
                    continue
            cur += ch
        if cur.strip():
            parts.append(cur)
        for part in parts:
            if ":" not in part:
                ok = False
                break
            k, v = part.split(":", 1)
            args[k.strip().strip('"')] = _loose_value(v)
        if ok:
            keep.append(text[pos:m.start()])
            pos = m.end()
            calls.append(_call(m.group(1), args))
    keep.append(text[pos:])
    return "".join(keep).strip(), calls


_DSML = "\uff5cDSML\uff5c"


def parse_deepseek_dsml(text: str) -> Tuple[str, List[dict]]:
    """``<|DSML|tool_calls> <|DSML|invoke name="f"> <|DSML|parameter name="k" string="true|false">v
    </|DSML|parameter> </|DSML|invoke> </|DSML|tool_calls>`` (full-width bars). An invoke with a
    repeated key or an unparsable non-string parameter is dropped whole."""
    o, c = f"<{_DSML}tool_calls>", f"</{_DSML}tool_calls>"
    i = text.find(o)
    if i < 0:
        return text, []
    j = text.find(c, i)
    block = text[i + len(o): j if j >= 0 else len(text)]
    calls = []
    for inv in re.finditer(rf'<{_DSML}invoke name="([^"]+)">(.*?)</{_DSML}invoke>', block, re.S):
        args, ok = {}, True
        for k, is_str, v in re.findall(rf'<{_DSML}parameter name="([^"]+)"(?: string="(true|false)")?>(.*?)</{_DSML}parameter>',
                                       inv.group(2), re.S):
            if k in args:
                ok = False
                break
            if is_str == "false":
                try:
                    args[k] = json.loads(v)
                except Exception:
                    ok = False
                    break
            else:
                args[k] = v
        if ok:
            calls.append(_call(inv.group(1), args))
    rest = (text[:i] + (text[j + len(c):] if j >= 0 else "")).strip()
    return (rest, calls) if calls else (text, [])


def parse_poolside_v1(text: str) -> Tuple[str, List[dict]]:
    """``<tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call>``; a bare NAME is a
    zero-argument call. Repeated keys or names that are not plain identifiers drop the call."""
    calls, keep, pos = [], [], 0
    for m in re.finditer(r"<tool_call>\s*([A-Za-z_][\w.\-]*)\s*((?:<arg_key>.*?</arg_key>\s*<arg_value>.*?</arg_value>\s*)*)</tool_call>",
                         text, re.S):
        args, ok = {}, True
        for k, v in re.findall(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", m.group(2), re.S):
            k = k.strip()
            if k in args or not re.fullmatch(r"[A-Za-z_][\w.\-]*", k):
                ok = False
                break
            args[k] = _loose_value(v)
        if ok:
            keep.append(text[pos:m.start()])
            pos = m.end()
            calls.append(_call(m.group(1), args))
    keep.append(text[pos:])
    return "".join(keep).strip(), calls


PARSERS = {"hermes": parse_hermes, "qwen3_xml": parse_qwen3_xml, "qwen3_coder": parse_qwen3_xml,
           "mistral": parse_mistral, "bare_json": parse_bare_json, "json": parse_bare_json,
           "minimax_xml": parse_minimax_xml, "gemma4": parse_gemma4, "deepseek_v4_dsml": parse_deepseek_dsml,
           "poolside_v1": parse_poolside_v1}
PIPELINE = {"hermes": ["hermes", "qwen3_xml", "bare_json"], "qwen3_xml": ["qwen3_xml", "hermes", "bare_json"],
            "qwen3_coder": ["qwen3_xml", "hermes", "bare_json"], "mistral": ["mistral", "bare_json"],
            "bare_json": ["bare_json"], "json": ["bare_json"],
            "minimax_xml": ["minimax_xml", "qwen3_xml", "hermes", "bare_json"], "gemma4": ["gemma4", "bare_json"],
            "deepseek_v4_dsml": ["deepseek_v4_dsml", "bare_json"],
            "poolside_v1": ["poolside_v1", "hermes", "bare_json"]}


def _coerce(value, schema: dict):
    t = (schema or {}).get("type")
    if isinstance(value, str):
        try:
            if t == "integer":
                return int(value)
            if t == "number":
                return float(value)
            if t == "boolean":
                return value.strip().lower() in ("true", "1", "yes")
            if t in ("object", "array"):
                return json.loads(value)
        except Exception:
            return value
    return value


def fix_calls(calls: List[dict], tools: Optional[List[dict]]) -> List[dict]:
    """Fuzzy-match tool names and coerce argument types to the declared JSON schema."""
    if not tools:
        return calls
    specs = {t["function"]["name"]: t["function"] for t in tools if t.get("type", "function") == "function"}
    out = []
    for c in calls:
        name = c["function"]["name"]
        if name not in specs:
            m = difflib.get_close_matches(name, list(specs), n=1, cutoff=0.6)
            if not m:
                continue
            name = m[0]
        try:
            args = json.loads(c["function"]["arguments"] or "{}")
        except Exception:
            args = {}
        props = (specs[name].get("parameters") or {}).get("properties", {})
        if isinstance(args, dict):
            args = {k: _coerce(v, props.get(k, {})) for k, v in args.items()}
        c = dict(c)
        c["function"] = {"name": name, "arguments": json.dumps(args, ensure_ascii=False)}
        out.append(c)
    return out


def parse_tool_calls(text: str, fmt: str = "hermes", tools: Optional[List[dict]] = None) -> Tuple[str, List[dict]]:
    """Primary parser for `fmt`, then salvage passes; reasoning before ``</think>`` is skipped."""
    head = ""
    i = text.find("</think>")
    if i >= 0:
        head, text = text[:i + len("</think>")], text[i + len("</think>"):]
    for name in PIPELINE.get(fmt, [fmt]):
        rest, calls = PARSERS[name](text)
        if calls:
            return head + rest, fix_calls(calls, tools)
    return head + text, []


class StreamingToolDetector:
    """Holds back streamed text from the first tool-call opener on, so clients never see raw
    call markup; the held text is parsed when the stream ends."""
    OPENERS = ("<tool_call>", "[TOOL_CALLS]", "<minimax:tool_call>", "<|tool_call>", "<\uff5cDSML\uff5ctool_calls>")

    def __init__(self):
        self.held = ""
        self.holding = False

    def push(self, text: str) -> str:
        if self.holding:
            self.held += text
            return ""
        buf = self.held + text
        for op in self.OPENERS:
            i = buf.find(op)
            if i >= 0:
                self.holding, self.held = True, buf[i:]
                return buf[:i]
        keep = 0
        for op in self.OPENERS:
            for k in range(min(len(op) - 1, len(buf)), 0, -1):
                if op.startswith(buf[-k:]):
                    keep = max(keep, k)
                    break
        self.held = buf[len(buf) - keep:] if keep else ""
        return buf[:len(buf) - keep] if keep else buf

    def finish(self) -> str:
        h, self.held = self.held, ""
        return h
