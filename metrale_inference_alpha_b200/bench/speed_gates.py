"""Latency measurements and their verdicts: a quick speed run, the TTFT gates with a stored per-host baseline, and
the boot-time memory check. Measuring and judging are separate functions; the judges do no I/O.

``quick_speed``    warm-up plus N timed runs of one prompt: the engine's decode rate ((completion tokens - 1) /
                   decode time, prefill excluded), TTFT and end-to-end rate. A measurement, not a gate. Each average
                   counts only the runs that reported its value.
``ttft_verdict``   a run's median and p90 TTFT against the stored baseline of the same host and model: pass within
                   the tolerance, fail beyond it, "no-baseline" when there is nothing usable to compare with (that
                   run becomes the baseline). A failed run never replaces the baseline.
``boot_memory``    what the engine holds on the device after a short warm-up wave (weights, KV pool blocks, ledger
                   total) against its memory budget; informational until a bound is given.

Reference: ``crates/bench/src/benchmarks/{quick_speed,ttft,ttft_verdict,ttft_target}.rs``, ``default_tier_boot/``.
"""
from __future__ import annotations

import json
import os
import statistics
import time
from typing import Dict, List, Optional, Sequence
from urllib.parse import urlsplit

from ..sampling.params import SamplingParams

_LOOPBACK = {"localhost", "127.0.0.1", "::1", "[::1]", "0.0.0.0"}


def same_host(a: str, b: str) -> bool:
    """Whether two endpoint URLs name the same server: loopback spellings are one host, a missing port is the
    scheme's default, paths and trailing slashes do not matter."""
    def norm(u: str):
        p = urlsplit(u if "://" in u else "http://" + u)
        host = (p.hostname or "").lower()
        host = "loopback" if host in _LOOPBACK else host
        return host, p.port or (443 if p.scheme == "https" else 80)
    return norm(a) == norm(b)


def _mean(xs: Sequence[Optional[float]]) -> Optional[float]:
    xs = [x for x in xs if x is not None]
    return sum(xs) / len(xs) if xs else None


def quick_speed(engine, prompt: Sequence[int], runs: int = 5, max_tokens: int = 64, warmup: int = 1) -> dict:
    rows = []
    for i in range(warmup + runs):
        t0 = time.perf_counter()
        out = engine.generate([list(prompt)], SamplingParams(max_tokens=max_tokens, temperature=0.0, ignore_eos=True))[0]
        wall = time.perf_counter() - t0
        if i < warmup:
            continue
        n = len(out.output_ids)
        dec = (n - 1) / (out.decode_ms / 1e3) if out.decode_ms and n > 1 else None
        rows.append({"decode_tok_s": dec, "ttft_ms": out.ttft_ms, "e2e_tok_s": n / wall if wall > 0 else None,
                     "tpot_ms": 1000.0 / dec if dec else None, "completion_tokens": n})
    return {"runs": rows, "decode_tok_s": _mean([r["decode_tok_s"] for r in rows]), "ttft_ms": _mean([r["ttft_ms"] for r in rows]),
            "e2e_tok_s": _mean([r["e2e_tok_s"] for r in rows]), "tpot_ms": _mean([r["tpot_ms"] for r in rows])}


# ----------------------------------------------------------------------------- TTFT gates
def summarise_ttft(samples_ms: Sequence[float]) -> dict:
    xs = sorted(x for x in samples_ms if x is not None)
    if not xs:
        return {"n": 0, "median_ms": None, "p90_ms": None}
    return {"n": len(xs), "median_ms": statistics.median(xs), "p90_ms": xs[min(len(xs) - 1, int(0.9 * len(xs)))]}


def ttft_verdict(run: dict, baseline: Optional[dict], tolerance: float = 0.10) -> dict:
    usable = lambda d: bool(d) and all(isinstance(d.get(k), (int, float)) and d[k] > 0 for k in ("median_ms", "p90_ms"))
    if not usable(run):
        return {"verdict": "fail", "should_store": False, "why": "the run has no usable median / p90"}
    if not usable(baseline):
        return {"verdict": "no-baseline", "should_store": True, "why": "nothing usable to compare with: this run becomes the baseline"}
    worse = [k for k in ("median_ms", "p90_ms") if run[k] > baseline[k] * (1.0 + tolerance)]
    if worse:
        return {"verdict": "fail", "should_store": False,
                "why": ", ".join(f"{k} {run[k]:.1f} against {baseline[k]:.1f} (+{100 * (run[k] / baseline[k] - 1):.0f} %)" for k in worse)}
    better = all(run[k] <= baseline[k] for k in ("median_ms", "p90_ms"))
    return {"verdict": "pass", "should_store": better, "why": ""}


class TtftBaselines:
    """Baselines in one JSON file, one entry per (host, model, warm | cold)."""

    def __init__(self, path: str):
        self.path = path
        self.data: List[dict] = json.load(open(path)) if os.path.exists(path) else []

    def find(self, url: str, model: str, kind: str) -> Optional[dict]:
        return next((e for e in self.data if e["model"] == model and e["kind"] == kind and same_host(e["url"], url)), None)

    def store(self, url: str, model: str, kind: str, summary: dict) -> None:
        self.data = [e for e in self.data if not (e["model"] == model and e["kind"] == kind and same_host(e["url"], url))]
        self.data.append({"url": url, "model": model, "kind": kind, **summary})
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.data, f, indent=1)
        os.replace(tmp, self.path)


def ttft_gate(engine, prompts: Sequence[Sequence[int]], baselines: TtftBaselines, kind: str = "cold", url: str = "in-process",
              tolerance: float = 0.10) -> dict:
    """``cold``: every prompt is new to the prefix cache. ``warm``: each prompt is sent once untimed first, so the
    timed request is a prefix hit."""
    if kind not in ("cold", "warm"):
        raise ValueError("kind must be cold | warm")
    sp = lambda: SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True)
    samples = []
    for p in prompts:
        if kind == "warm":
            engine.generate([list(p)], sp())
        samples.append(engine.generate([list(p)], sp())[0].ttft_ms)
    run = summarise_ttft(samples)
    res = ttft_verdict(run, baselines.find(url, engine.cfg.name, kind), tolerance)
    if res["should_store"]:
        baselines.store(url, engine.cfg.name, kind, run)
    return {**run, **res, "kind": kind}


# ----------------------------------------------------------------------------- boot memory
def boot_memory(engine, budget_bytes: Optional[int] = None, warmup_prompts: Sequence[Sequence[int]] = ()) -> dict:
    if warmup_prompts:
        engine.generate([list(p) for p in warmup_prompts], [SamplingParams(max_tokens=4, temperature=0.0) for _ in warmup_prompts])
    st, mem = engine.stats(), engine.memory_report()
    held = mem["ledger_bytes"] + st["weights_bytes"]
    out = {"kv_blocks": st["kv_blocks"], "weights_bytes": st["weights_bytes"], "ledger_bytes": mem["ledger_bytes"],
           "slack_bytes": mem["slack_bytes"], "held_bytes": held, "budget_bytes": budget_bytes}
    out["verdict"] = "info" if budget_bytes is None else ("pass" if held <= budget_bytes else "fail")
    return out
