"""Two serving-correctness suites that need no reference answers.

``contamination``: concurrent requests each carry a distinct secret in their prompt; a response that
contains another request's secret means state leaked between sequences (a KV block, a recurrent-state
slot or a sampler buffer shared by mistake). The prompts share a long common prefix so the prefix cache
and block sharing are exercised, and the run is repeated under churn (requests of different lengths
finishing at different times, so blocks are recycled while neighbours still decode).

``scheduler_equivalence``: the same greedy requests must produce the same tokens whatever the scheduling
— admission policy, chunked-prefill budget, batch cap, arrival order — because scheduling decides only
when a token is computed. Each variant is compared with a baseline run token by token; the report names
the first diverging position per request.

Reference: ``crates/bench/src/benchmarks/{contamination,scheduler_equivalence}``.
"""
from __future__ import annotations

import random
from typing import Callable, Dict, List, Optional, Sequence


# ----------------------------------------------------------------------------- contamination
def contamination(engine, tokenizer=None, n_requests: int = 8, rounds: int = 2, prefix_tokens: int = 48, max_tokens: int = 24,
                  seed: int = 0) -> dict:
    """Token-level form for an in-process engine: every request's prompt = a shared prefix + a block of
    16 ids unique to the request (its "secret", drawn from an id range nothing else uses). A response
    reproducing 4 or more consecutive ids of another request's secret is a leak. Returns
    ``{"requests", "leaks": [...], "ok"}``."""
    from ..sampling.params import SamplingParams
    rng = random.Random(seed)
    vocab = engine.cfg.vocab_size
    lo = vocab // 2
    span = (vocab - lo) // (n_requests * rounds + 1)
    if span < 16:
        raise ValueError("vocabulary too small for this many distinct secrets")
    prefix = [rng.randrange(3, lo) for _ in range(prefix_tokens)]
    leaks, total = [], 0
    for r in range(rounds):
        secrets = [[lo + (r * n_requests + i) * span + j for j in range(16)] for i in range(n_requests)]
        prompts = [prefix + s + [rng.randrange(3, lo) for _ in range(rng.randrange(1, 9))] for s in secrets]
        params = [SamplingParams(max_tokens=max_tokens + 3 * (i % 4), temperature=0.0) for i in range(n_requests)]
        outs = engine.generate(prompts, params)
        total += len(outs)
        for i, o in enumerate(outs):
            ids = o.output_ids
            for j, s in enumerate(secrets):
                if j == i:
                    continue
                grams = {tuple(s[k:k + 4]) for k in range(len(s) - 3)}
                if any(tuple(ids[k:k + 4]) in grams for k in range(len(ids) - 3)):
                    leaks.append({"round": r, "request": i, "secret_of": j})
    return {"requests": total, "leaks": leaks, "ok": not leaks}


# ----------------------------------------------------------------------------- scheduler equivalence
def scheduler_equivalence(make_engine: Callable[..., object], variants: Optional[Dict[str, dict]] = None, n: int = 6,
                          prompt_len: int = 40, max_tokens: int = 16, seed: int = 0) -> dict:
    """``make_engine(**overrides)`` builds an engine; the baseline uses no overrides. Returns per variant
    whether every request's tokens equal the baseline's and, if not, where they first differ."""
    from ..sampling.params import SamplingParams
    variants = variants if variants is not None else {
        "small_prefill_chunks": {"max_prefill_tokens": 16},
        "batch_cap_2": {"max_num_seqs": 2},
        "tbt_policy": {"scheduler": "tbt"},
        "no_prefix_cache": {"enable_prefix_caching": False},
    }
    rng = random.Random(seed)
    base = make_engine()
    vocab = base.cfg.vocab_size
    shared = [rng.randrange(3, vocab) for _ in range(prompt_len // 2)]
    prompts = [shared + [rng.randrange(3, vocab) for _ in range(prompt_len // 2 + i)] for i in range(n)]
    sp = SamplingParams(max_tokens=max_tokens, temperature=0.0)
    want = [o.output_ids for o in base.generate(prompts, sp)]
    report = {}
    for name, kw in variants.items():
        eng = make_engine(**kw)
        order = list(range(n))
        random.Random(seed + 1).shuffle(order)                   # arrival order is part of the schedule
        outs = eng.generate([prompts[i] for i in order], sp)
        got = [None] * n
        for slot, i in enumerate(order):
            got[i] = outs[slot].output_ids
        diffs = []
        for i in range(n):
            if got[i] != want[i]:
                pos = next((k for k, (a, b) in enumerate(zip(got[i], want[i])) if a != b), min(len(got[i]), len(want[i])))
                diffs.append({"request": i, "first_difference": pos})
        report[name] = {"equal": not diffs, "differences": diffs}
    return {"variants": report, "ok": all(v["equal"] for v in report.values())}
