"""Concurrency ladder through the public engine API: for each rung C, C requests of ISL random
token ids arrive at once, greedy, OSL new tokens each with EOS ignored; reports aggregate
decode tokens/s, TTFT percentiles and ms/step. Same workload definition as the reference's
certification ladder (``scripts/bench_concurrency_ladder.py``, ISL128 / OSL1024, rungs
1..128, prompts from seed 42), driven in-process instead of over HTTP.
"""
from __future__ import annotations

import random
import statistics
import time
from typing import List

import torch

from ..engine.llm_engine import EngineArgs, LLMEngine
from ..sampling.params import SamplingParams


def _pct(xs: List[float], q: float) -> float:
    if not xs:
        return float("nan")
    xs = sorted(xs)
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


def run_rung(engine: LLMEngine, concurrency: int, isl: int, osl: int, seed: int = 42) -> dict:
    rng = random.Random(seed + concurrency)
    vocab = engine.cfg.vocab_size
    sp = SamplingParams(max_tokens=osl, temperature=0.0, ignore_eos=True)
    cuda = engine.device.type == "cuda"
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    sync()
    t0 = time.perf_counter()
    first = {}
    ids = [engine.add_request([rng.randrange(1, vocab) for _ in range(isl)], sp) for _ in range(concurrency)]
    tokens, steps, t_decode0, tokens_at_decode0 = 0, 0, None, 0
    while engine.has_work():
        outs = engine.step()
        steps += 1
        now = time.perf_counter()
        for o in outs:
            if o.new_token_ids and o.request_id not in first:
                first[o.request_id] = now - t0
            tokens += len(o.new_token_ids)
        if t_decode0 is None and len(first) == concurrency:
            t_decode0, tokens_at_decode0, steps_at_decode0 = now, tokens, steps
    sync()
    t1 = time.perf_counter()
    ttft = [first[i] * 1e3 for i in ids if i in first]
    dec_tokens = tokens - tokens_at_decode0
    dec_s = max(t1 - (t_decode0 or t0), 1e-9)
    return {"concurrency": concurrency, "isl": isl, "osl": osl, "tokens": tokens,
            "tok_s": tokens / (t1 - t0), "decode_tok_s": dec_tokens / dec_s,
            "ttft_p50_ms": _pct(ttft, 0.5), "ttft_p99_ms": _pct(ttft, 0.99),
            "ttft_mean_ms": statistics.fmean(ttft) if ttft else float("nan"),
            "ms_per_step": dec_s * 1e3 / max(1, steps - (steps_at_decode0 if t_decode0 else 0)),
            "steps": steps, "wall_s": t1 - t0}


def run_ladder(args: EngineArgs, rungs: List[int], isl: int = 128, osl: int = 1024, warmup: bool = True) -> List[dict]:
    args.max_num_seqs = max(args.max_num_seqs, max(rungs))
    args.max_model_len = max(args.max_model_len, isl + osl + 16)
    engine = LLMEngine(args)
    rows = []
    for c in rungs:
        if warmup:                               # graph capture and allocator warm-up for this rung
            run_rung(engine, c, min(isl, 16), 4, seed=7)
        rows.append(run_rung(engine, c, isl, osl))
    return rows
