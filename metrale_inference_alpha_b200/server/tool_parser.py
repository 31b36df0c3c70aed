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


PARSERS = {"hermes": parse_hermes, "qwen3_xml": parse_qwen3_xml, "qwen3_coder": parse_qwen3_xml,
           "mistral": parse_mistral, "bare_json": parse_bare_json}
PIPELINE = {"hermes": ["hermes", "qwen3_xml", "bare_json"], "qwen3_xml": ["qwen3_xml", "hermes", "bare_json"],
            "qwen3_coder": ["qwen3_xml", "hermes", "bare_json"], "mistral": ["mistral", "bare_json"],
            "bare_json": ["bare_json"]}


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
    OPENERS = ("<tool_call>", "[TOOL_CALLS]")

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
