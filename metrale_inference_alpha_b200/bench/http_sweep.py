"""Concurrency sweep against a running server over HTTP: for each rung C, C streaming chat
requests start together (prompts of ISL random words from a seeded generator, ``max_tokens`` = OSL,
``ignore_eos`` through ``min_tokens``), and the client records per request the time to the first
content chunk, the inter-chunk gaps and the usage block the server reports. Output per rung:
aggregate completion tokens / wall second, TTFT p50 / p99 as seen by the client, the server's own
``time_to_first_token_ms`` p50, mean time per output token, errors.

This is the over-the-wire form of the certification ladder (role of the reference's
``scripts/bench_concurrency_ladder.py`` and the SSE client of ``crates/bench/src/http``); the
in-process form is ``bench/ladder.py``.
"""
from __future__ import annotations

import asyncio
import json
import random
import time
from typing import Dict, List, Optional

_WORDS = ("alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu nu xi omicron pi rho sigma tau "
          "upsilon phi chi psi omega").split()


def _pct(xs: List[float], q: float) -> Optional[float]:
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))]


def make_prompt(rng: random.Random, words: int) -> str:
    return " ".join(rng.choice(_WORDS) for _ in range(words))


async def one_request(session, url: str, body: dict, headers: Dict[str, str]) -> dict:
    t0 = time.perf_counter()
    first, last, gaps, usage, chunks, err = None, None, [], None, 0, None
    try:
        async with session.post(url + "/v1/chat/completions", json=body, headers=headers) as r:
            if r.status != 200:
                return {"error": f"HTTP {r.status}: {(await r.text())[:200]}", "seconds": time.perf_counter() - t0}
            async for raw in r.content:
                line = raw.decode("utf-8", "replace").strip()
                if not line.startswith("data: "):
                    continue
                data = line[6:]
                if data == "[DONE]":
                    break
                d = json.loads(data)
                if "error" in d:
                    err = str(d["error"].get("message"))
                    break
                if d.get("usage"):
                    usage = d["usage"]
                for ch in d.get("choices") or []:
                    delta = ch.get("delta") or {}
                    # every chunk after the opening role chunk carries newly decoded tokens (its text
                    # may be empty while a multi-byte character is still incomplete)
                    if "role" not in delta:
                        now = time.perf_counter()
                        if first is None:
                            first = now
                        else:
                            gaps.append(now - last)
                        last = now
                        chunks += 1
    except Exception as e:                                   # connection errors are results, not crashes
        err = f"{type(e).__name__}: {e}"
    out = {"seconds": time.perf_counter() - t0, "ttft_ms": None if first is None else (first - t0) * 1e3,
           "chunks": chunks, "gaps": gaps, "usage": usage}
    if err:
        out["error"] = err
    return out


async def run_rung(url: str, concurrency: int, isl_words: int, osl: int, model: str = "default",
                   api_key: Optional[str] = None, seed: int = 42, temperature: float = 0.0) -> dict:
    import aiohttp
    rng = random.Random(seed + concurrency)
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    bodies = [{"model": model, "messages": [{"role": "user", "content": make_prompt(rng, isl_words)}], "stream": True,
               "stream_options": {"include_usage": True}, "max_tokens": osl, "min_tokens": osl, "temperature": temperature}
              for _ in range(concurrency)]
    timeout = aiohttp.ClientTimeout(total=None, sock_read=600)
    async with aiohttp.ClientSession(timeout=timeout, connector=aiohttp.TCPConnector(limit=0)) as s:
        t0 = time.perf_counter()
        res = await asyncio.gather(*(one_request(s, url.rstrip("/"), b, headers) for b in bodies))
        wall = time.perf_counter() - t0
    ok = [r for r in res if "error" not in r]
    toks = sum(int((r["usage"] or {}).get("completion_tokens") or 0) for r in ok)
    gaps = [g for r in ok for g in r["gaps"]]
    return {"concurrency": concurrency, "requests": len(res), "errors": len(res) - len(ok),
            "first_error": next((r["error"] for r in res if "error" in r), None),
            "completion_tokens": toks, "wall_s": wall, "tok_s": toks / wall if wall > 0 else 0.0,
            "ttft_p50_ms": _pct([r["ttft_ms"] for r in ok if r["ttft_ms"] is not None], 0.5),
            "ttft_p99_ms": _pct([r["ttft_ms"] for r in ok if r["ttft_ms"] is not None], 0.99),
            "server_ttft_p50_ms": _pct([float(r["usage"]["time_to_first_token_ms"]) for r in ok
                                        if r["usage"] and r["usage"].get("time_to_first_token_ms") is not None], 0.5),
            "chunk_gap_ms_mean": (1e3 * sum(gaps) / len(gaps)) if gaps else None}


def run_sweep(url: str, rungs: List[int], isl_words: int = 96, osl: int = 128, **kw) -> List[dict]:
    return [asyncio.run(run_rung(url, c, isl_words, osl, **kw)) for c in rungs]
