"""Function-calling benchmark in the style of BFCL single-turn: draw samples, ask the served model for a
tool call, and check the call against the sample's ground truth with an AST-style matcher.

Dataset: JSONL, one sample per line::

    {"id": "simple_12", "category": "simple", "question": [{"role": "user", "content": "..."}],
     "functions": [<JSON-schema function specs>],
     "ground_truth": [{"get_weather": {"city": ["Paris", "paris"], "unit": ["celsius", ""]}}]}

``ground_truth`` lists the expected calls (several for the parallel categories); each parameter maps to
the list of accepted values, where ``""`` in the list marks the parameter as optional. The checker
accepts a call when the function name matches, no unknown or missing required parameter appears, and
every given value equals an accepted one after the usual coercions (ints for floats, case-insensitive
strings without surrounding blanks, lists and dicts element by element). ``irrelevance`` samples expect
no call at all.

The draw is deterministic (``seed``), optionally a subset (``n``) and optionally one shard of several, so a
run reports its size before generating; generation sends one sample at a time through ``ask`` (any
callable ``(messages, tools) -> assistant message dict`` — ``http_asker`` builds one for an
OpenAI-compatible endpoint, ``app_asker`` for an in-process FastAPI app). A few built-in samples serve as
a smoke set; real suites point ``load_dataset`` at their own file.

Reference: ``crates/bench/src/benchmarks/bfcl/{dataset,draw,exec,aggregate,report}.rs`` (there the
ground truth and the checker live in an external Python package).
"""
from __future__ import annotations

import json
import random
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

Asker = Callable[[List[dict], List[dict]], dict]


@dataclass
class Sample:
    id: str
    category: str
    question: List[dict]
    functions: List[dict]
    ground_truth: List[Dict[str, Dict[str, list]]]


@dataclass
class Verdict:
    id: str
    category: str
    ok: bool
    reason: str = ""
    calls: List[dict] = field(default_factory=list)


SMOKE_SET = [
    {"id": "simple_0", "category": "simple",
     "question": [{"role": "user", "content": "What is the weather in Paris in celsius?"}],
     "functions": [{"name": "get_weather", "description": "Current weather of a city.",
                    "parameters": {"type": "object", "properties": {"city": {"type": "string"}, "unit": {"type": "string", "enum": ["celsius", "fahrenheit"]}},
                                   "required": ["city"]}}],
     "ground_truth": [{"get_weather": {"city": ["Paris"], "unit": ["celsius", ""]}}]},
    {"id": "simple_1", "category": "simple",
     "question": [{"role": "user", "content": "Compute the area of a triangle with base 10 and height 5."}],
     "functions": [{"name": "triangle_area", "description": "Area of a triangle.",
                    "parameters": {"type": "object", "properties": {"base": {"type": "number"}, "height": {"type": "number"}},
                                   "required": ["base", "height"]}}],
     "ground_truth": [{"triangle_area": {"base": [10], "height": [5]}}]},
    {"id": "multiple_0", "category": "multiple",
     "question": [{"role": "user", "content": "Convert 100 USD to EUR."}],
     "functions": [{"name": "convert_currency", "description": "Convert an amount between currencies.",
                    "parameters": {"type": "object", "properties": {"amount": {"type": "number"}, "from": {"type": "string"}, "to": {"type": "string"}},
                                   "required": ["amount", "from", "to"]}},
                   {"name": "get_stock_price", "description": "Price of a stock.",
                    "parameters": {"type": "object", "properties": {"symbol": {"type": "string"}}, "required": ["symbol"]}}],
     "ground_truth": [{"convert_currency": {"amount": [100], "from": ["USD"], "to": ["EUR"]}}]},
    {"id": "parallel_0", "category": "parallel",
     "question": [{"role": "user", "content": "Weather in Rome and in Oslo?"}],
     "functions": [{"name": "get_weather", "description": "Current weather of a city.",
                    "parameters": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}],
     "ground_truth": [{"get_weather": {"city": ["Rome"]}}, {"get_weather": {"city": ["Oslo"]}}]},
    {"id": "irrelevance_0", "category": "irrelevance",
     "question": [{"role": "user", "content": "Tell me a joke about compilers."}],
     "functions": [{"name": "get_weather", "description": "Current weather of a city.",
                    "parameters": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}],
     "ground_truth": []},
]


def load_dataset(path: Optional[str] = None) -> List[Sample]:
    rows = SMOKE_SET if path is None else [json.loads(l) for l in open(path) if l.strip()]
    out = []
    for r in rows:
        if not {"id", "question", "functions", "ground_truth"} <= set(r):
            raise ValueError(f"sample {r.get('id')!r} lacks a required field")
        out.append(Sample(r["id"], r.get("category") or r["id"].rsplit("_", 1)[0], r["question"], r["functions"], r["ground_truth"]))
    return out


def draw(samples: Sequence[Sample], n: Optional[int] = None, seed: int = 0, shard: int = 0, shards: int = 1) -> List[Sample]:
    """Deterministic subset: a seeded shuffle stratified by category (so a subset keeps every category in
    proportion), then shard ``shard`` of ``shards`` by stride."""
    if not 0 <= shard < shards:
        raise ValueError("shard index out of range")
    by_cat: Dict[str, List[Sample]] = {}
    for s in sorted(samples, key=lambda s: s.id):
        by_cat.setdefault(s.category, []).append(s)
    rng = random.Random(seed)
    for v in by_cat.values():
        rng.shuffle(v)
    total = sum(len(v) for v in by_cat.values())
    n = total if n is None else min(n, total)
    picked: List[Sample] = []
    cats = sorted(by_cat)
    quota = {c: (len(by_cat[c]) * n) // total for c in cats}
    rest = n - sum(quota.values())
    for c in sorted(cats, key=lambda c: -((len(by_cat[c]) * n) % total))[:rest]:
        quota[c] += 1
    for c in cats:
        picked += by_cat[c][:quota[c]]
    picked.sort(key=lambda s: s.id)
    return picked[shard::shards]


# ----------------------------------------------------------------------------- checker
def _norm(v):
    if isinstance(v, str):
        return v.strip().lower()
    if isinstance(v, bool):
        return v
    if isinstance(v, (int, float)):
        return float(v)
    if isinstance(v, list):
        return [_norm(x) for x in v]
    if isinstance(v, dict):
        return {k: _norm(x) for k, x in v.items()}
    return v


def _value_ok(given, accepted: list) -> bool:
    g = _norm(given)
    for a in accepted:
        if a == "" and not isinstance(given, str):
            continue
        if _norm(a) == g:
            return True
        if isinstance(a, str) and isinstance(given, (int, float)) and not isinstance(given, bool):
            try:
                if float(a) == float(given):
                    return True
            except ValueError:
                pass
    return False


def check_call(call: dict, expected: Dict[str, Dict[str, list]], spec: Optional[dict] = None) -> str:
    """'' when ``call`` ({"name", "arguments"}) matches ``expected`` ({name: {param: accepted}}), else why not."""
    (name, params), = expected.items()
    if call.get("name") != name:
        return f"function {call.get('name')!r}, expected {name!r}"
    args = call.get("arguments")
    if isinstance(args, str):
        try:
            args = json.loads(args)
        except ValueError:
            return "arguments are not JSON"
    if not isinstance(args, dict):
        return "arguments are not an object"
    for k in args:
        if k not in params:
            return f"unexpected parameter {k!r}"
    required = set((spec or {}).get("parameters", {}).get("required", []))
    for k, accepted in params.items():
        if k not in args:
            if "" in accepted and k not in required:
                continue
            return f"missing parameter {k!r}"
        if not _value_ok(args[k], accepted):
            return f"parameter {k!r} = {args[k]!r} is not one of {accepted!r}"
    return ""


def check_sample(sample: Sample, calls: List[dict]) -> Verdict:
    specs = {f["name"]: f for f in sample.functions}
    if not sample.ground_truth:
        return Verdict(sample.id, sample.category, not calls, "" if not calls else "a call where none was relevant", calls)
    if len(calls) != len(sample.ground_truth):
        return Verdict(sample.id, sample.category, False, f"{len(calls)} calls, expected {len(sample.ground_truth)}", calls)
    # order-free matching (parallel categories): every expected call must claim a distinct produced call
    left = list(calls)
    why = ""
    for exp in sample.ground_truth:
        hit = None
        for c in left:
            why = check_call(c, exp, specs.get(next(iter(exp))))
            if not why:
                hit = c
                break
        if hit is None:
            return Verdict(sample.id, sample.category, False, why, calls)
        left.remove(hit)
    return Verdict(sample.id, sample.category, True, "", calls)


def calls_of_message(msg: dict) -> List[dict]:
    out = []
    for tc in msg.get("tool_calls") or []:
        f = tc.get("function", tc)
        out.append({"name": f.get("name"), "arguments": f.get("arguments")})
    return out


# ----------------------------------------------------------------------------- run / aggregate
def run(samples: Sequence[Sample], ask: Asker, on_progress: Optional[Callable[[int, int], None]] = None,
        should_stop: Optional[Callable[[], bool]] = None) -> List[Verdict]:
    out = []
    for i, s in enumerate(samples):
        if should_stop and should_stop():
            break
        tools = [{"type": "function", "function": f} for f in s.functions]
        try:
            msg = ask(s.question, tools)
            out.append(check_sample(s, calls_of_message(msg)))
        except Exception as e:                  # a failed request is a failed sample, not a failed run
            out.append(Verdict(s.id, s.category, False, f"request failed: {e}"))
        if on_progress:
            on_progress(i + 1, len(samples))
    return out


def aggregate(verdicts: Sequence[Verdict]) -> dict:
    cats: Dict[str, List[Verdict]] = {}
    for v in verdicts:
        cats.setdefault(v.category, []).append(v)
    per = {c: {"n": len(v), "correct": sum(x.ok for x in v), "accuracy": sum(x.ok for x in v) / len(v)} for c, v in sorted(cats.items())}
    n = len(verdicts)
    return {"n": n, "correct": sum(v.ok for v in verdicts), "accuracy": (sum(v.ok for v in verdicts) / n) if n else 0.0,
            "macro_accuracy": (sum(p["accuracy"] for p in per.values()) / len(per)) if per else 0.0, "categories": per,
            "failures": [{"id": v.id, "reason": v.reason} for v in verdicts if not v.ok]}


def report(agg: dict) -> str:
    lines = [f"function calling: {agg['correct']} / {agg['n']} = {agg['accuracy']:.1%} (macro {agg['macro_accuracy']:.1%})"]
    for c, p in agg["categories"].items():
        lines.append(f"  {c:<14} {p['correct']:>4} / {p['n']:<4} {p['accuracy']:.1%}")
    for f in agg["failures"][:10]:
        lines.append(f"  x {f['id']}: {f['reason']}")
    return "\n".join(lines)


def app_asker(client, model: str = "default", max_tokens: int = 256, **extra) -> Asker:
    """Asker over a ``fastapi.testclient.TestClient`` (or anything with ``.post(path, json=)``)."""
    def ask(messages, tools):
        r = client.post("/v1/chat/completions", json=dict(model=model, messages=messages, tools=tools, temperature=0,
                                                          max_tokens=max_tokens, **extra))
        if r.status_code != 200:
            raise RuntimeError(f"HTTP {r.status_code}: {r.text[:200]}")
        return r.json()["choices"][0]["message"]
    return ask


def http_asker(url: str, model: str = "default", api_key: Optional[str] = None, max_tokens: int = 256, timeout: float = 300.0) -> Asker:
    import requests

    def ask(messages, tools):
        h = {"Authorization": f"Bearer {api_key}"} if api_key else {}
        r = requests.post(url.rstrip("/") + "/v1/chat/completions", headers=h, timeout=timeout,
                          json=dict(model=model, messages=messages, tools=tools, temperature=0, max_tokens=max_tokens))
        r.raise_for_status()
        return r.json()["choices"][0]["message"]
    return ask
