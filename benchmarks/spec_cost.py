"""What one speculative step costs next to a plain decode step (``python -m benchmarks.spec_cost``).

One engine with a multi-token-prediction head (random weights of the named architecture, so
drafts are rejected and every verify step commits exactly one token: the measurement is the cost
side of speculation only). At batch C it times, through the engine's own step loop,
  * plain decode steps (graph replay, one-step look-ahead), and
  * for K = 1..4: the verify step over C x (K + 1) rows and the K-step draft proposal,
each with a device synchronisation on both sides. Role of the reference's gate statistics, which
compare these same two step times (``crates/server/src/scheduler/mtp_gate.rs``).
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def run(model: str, device: str, C: int = 8, ks=(1, 2, 3, 4), steps: int = 32, isl: int = 128,
        ctx_len: int = 2048) -> dict:
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.speculative.ladder import KLadder

    cfg = preset(model, mtp_layers=1)
    eng = LLMEngine(EngineArgs(model=cfg, device=device, max_num_seqs=max(C, 8), max_model_len=ctx_len,
                               speculative="mtp", num_drafts=max(ks), mtp_gate=False,
                               enable_prefix_caching=False, gpu_memory_utilization=0.85, seed=0))
    g = torch.Generator().manual_seed(7)
    sp = SamplingParams(max_tokens=ctx_len - isl - 8, temperature=0.0, ignore_eos=True)
    for _ in range(C):
        eng.add_request(torch.randint(0, cfg.vocab_size, (isl,), generator=g).tolist(), sp)
    while eng.scheduler.waiting or eng.scheduler.prefilling:
        eng.step()
    runner = eng.runner
    acc = {"verify": 0.0, "propose": 0.0}
    real_execute, real_propose = runner.execute, runner.propose

    def timed(name, fn):
        def wrapped(*a, **kw):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = fn(*a, **kw)
            torch.cuda.synchronize()
            acc[name] += time.perf_counter() - t0
            return out
        return wrapped

    def loop(n):
        torch.cuda.synchronize()
        tok0 = eng.scheduler.stats["decode_tokens"]
        t0 = time.perf_counter()
        for _ in range(n):
            eng.step()
        eng.flush()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / n * 1e3, (eng.scheduler.stats["decode_tokens"] - tok0) / n

    out = {"model": model, "concurrency": C, "steps": steps, "context": isl}
    eng.spec_mode = "none"
    loop(6)
    out["decode_ms"], _ = loop(steps)
    rows = []
    for K in ks:
        eng.flush()
        eng.spec_mode = "mtp"
        eng.ladder = KLadder(spec=f"{1 << 20}:{K}", max_k=K)
        runner.execute, runner.propose = real_execute, real_propose
        loop(6)                                             # first steps capture the (rung, K) graphs
        acc["verify"] = acc["propose"] = 0.0
        runner.execute, runner.propose = timed("verify", real_execute), timed("propose", real_propose)
        l0 = runner.graph_replays
        ms, toks = loop(steps)
        rows.append({"K": K, "step_ms": round(ms, 3), "verify_ms": round(acc["verify"] / steps * 1e3, 3),
                     "propose_ms": round(acc["propose"] / steps * 1e3, 3),
                     "verify_over_decode": round(acc["verify"] / steps * 1e3 / out["decode_ms"], 3),
                     # tokens a sequence must commit per speculative step (accepted drafts + 1) to match plain decode
                     "break_even_accept_len": round(ms / out["decode_ms"], 3),
                     "tokens_per_step": round(toks, 2), "graph_replays_per_step": (runner.graph_replays - l0) / steps})
    runner.execute, runner.propose = real_execute, real_propose
    out["decode_ms"] = round(out["decode_ms"], 3)
    out["by_k"] = rows
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense-27b-nvfp4")
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--isl", type=int, default=128)
    a = ap.parse_args()
    print(json.dumps(run(a.model, "cuda:0", a.concurrency, steps=a.steps, isl=a.isl)))


if __name__ == "__main__":
    main()
