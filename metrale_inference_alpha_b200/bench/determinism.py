"""Determinism gates over the public engine API.

* `kat_equality`: a fixed set of requests ("known answers") must produce byte-identical output
  whatever the engine did before: on a fresh engine, after unrelated traffic has filled the prefix
  cache and recycled KV blocks, and when the same request is repeated (prefix-cache hit). Role of
  the reference's ``kat-equality-gate`` ("same sample -> same bytes regardless of history",
  ``crates/bench`` kat_equality).
* `state_poisoning`: on models with recurrent layers, one request is replayed N times (12 in the
  reference) with other requests in between that dirty the recycled state slots and snapshot area;
  every replay must equal the first. Role of the ``ssm-state-poisoning-gate``.

Both return a `GateRecord` (value 1.0 = pass) whose config names the first mismatch, so they plug
into the same signing / ledger path as the throughput gates.
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch

from ..sampling.params import SamplingParams
from .gate import GateRecord, kernel_closure_hash


def _prompts(vocab: int, n: int, length: int, seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(1, vocab, (length + 3 * i,), generator=g).tolist() for i in range(n)]


def _run(engine, prompts: Sequence[Sequence[int]], max_tokens: int, seeded: bool) -> List[List[int]]:
    sps = [SamplingParams(max_tokens=max_tokens, temperature=0.8 if seeded else 0.0, top_p=0.9 if seeded else 1.0,
                          seed=1234 + len(p) if seeded else None, ignore_eos=True) for p in prompts]
    return [o.output_ids for o in engine.generate(prompts, sps)]


def kat_equality(make_engine: Callable[[], object], n: int = 4, prompt_len: int = 40, max_tokens: int = 24,
                 seeded: bool = False, device: str = "") -> GateRecord:
    eng = make_engine()
    vocab = eng.cfg.vocab_size
    kat = _prompts(vocab, n, prompt_len, seed=11)
    want = [_run(eng, [p], max_tokens, seeded)[0] for p in kat]             # fresh engine, one at a time
    bad = ""
    eng2 = make_engine()
    _run(eng2, _prompts(vocab, 6, prompt_len + 9, seed=99), max_tokens, False)   # unrelated history
    # second pass: the same requests again, now prefix-cache hits. A hit prefills fewer rows, which
    # changes the GEMM shapes and with them the rounding of the logits by an ulp: greedy answers
    # must survive that, sampled ones (a near-tie in the sorted tail flips the pick) are only
    # compared on the first pass
    for rep in range(1 if seeded else 2):
        for i, p in enumerate(kat):
            got = _run(eng2, [p], max_tokens, seeded)[0]
            if got != want[i] and not bad:
                k = next((j for j, (a, b) in enumerate(zip(got, want[i])) if a != b), min(len(got), len(want[i])))
                bad = f"request {i}, pass {rep}, first difference at output token {k}"
    return GateRecord("kat-equality", "same request -> same tokens regardless of history", 0.0 if bad else 1.0, "pass",
                      config={"requests": n, "prompt_len": prompt_len, "max_tokens": max_tokens, "seeded_sampling": seeded,
                              "mismatch": bad, "model": eng.cfg.name}, closure=kernel_closure_hash(), device=device)


def state_poisoning(make_engine: Callable[[], object], replays: int = 12, prompt_len: int = 48, max_tokens: int = 16,
                    device: str = "") -> GateRecord:
    eng = make_engine()
    vocab = eng.cfg.vocab_size
    probe = _prompts(vocab, 1, prompt_len, seed=21)[0]
    noise = _prompts(vocab, 3 * replays, prompt_len // 2, seed=22)
    first = _run(eng, [probe], max_tokens, False)[0]
    bad = ""
    for r in range(replays):
        _run(eng, noise[3 * r:3 * r + 3], max_tokens // 2, False)           # recycles state slots and snapshots
        got = _run(eng, [probe], max_tokens, False)[0]
        if got != first and not bad:
            bad = f"replay {r + 1} differs from the first run"
    return GateRecord("ssm-state-poisoning", f"{replays} replays byte-identical", 0.0 if bad else 1.0, "pass",
                      config={"replays": replays, "recurrent_layers": eng.runner.pool.num_layers if eng.runner.pool else 0,
                              "mismatch": bad, "model": eng.cfg.name}, closure=kernel_closure_hash(), device=device)
