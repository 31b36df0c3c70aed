#!/usr/bin/env python
"""One decode step of a model at concurrency C, run eagerly between cudaProfilerStart / cudaProfilerStop, so that a
launch list of exactly that step can be taken:

    python benchmarks/step_launches.py --model qwen-hybrid-moe-35b-fp8 --concurrency 128 &&
    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv \\
        --log-file launches.csv python benchmarks/step_launches.py --model qwen-hybrid-moe-35b-fp8 --concurrency 128

(one pass per launch: nothing is saved or restored around the kernels). `--summarise launches.csv` prints the
per-kernel totals of such a file and needs no GPU. Synthetic weights of the named architecture, random prompts.
"""
from __future__ import annotations

import argparse
import csv
import os
import re
import sys
from collections import defaultdict

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def summarise(path: str) -> None:
    rows = [r for r in csv.reader(open(path)) if len(r) > 10]
    hdr = rows[0]
    ki, vi = hdr.index("Kernel Name"), hdr.index("Metric Value")
    tot, cnt = defaultdict(float), defaultdict(int)
    for r in rows[1:]:
        name = re.sub(r"\(.*", "", r[ki]).replace("void ", "").replace("<unnamed>::", "")
        tot[name] += float(r[vi].replace(",", "")) / 1e3
        cnt[name] += 1
    whole = sum(tot.values())
    print(f"{len(rows) - 1} launches, {whole:.1f} us in kernels")
    for name, t in sorted(tot.items(), key=lambda kv: -kv[1]):
        print(f"{t:10.1f} us  {100 * t / whole:5.1f} %  x{cnt[name]:<5d} {name[:90]}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense-27b-nvfp4")
    ap.add_argument("--concurrency", type=int, default=128)
    ap.add_argument("--isl", type=int, default=128)
    ap.add_argument("--decode-steps", type=int, default=4, help="eager decode steps before the profiled one")
    ap.add_argument("--summarise", default=None)
    ns = ap.parse_args()
    if ns.summarise:
        return summarise(ns.summarise)
    import torch

    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    cfg = preset(ns.model)
    eng = LLMEngine(EngineArgs(model=cfg, device="cuda", max_num_seqs=128, max_model_len=ns.isl + 64,
                               max_prefill_tokens=8192, gpu_memory_utilization=0.85, use_cuda_graphs=False, seed=0))
    g = torch.Generator().manual_seed(42)
    sp = SamplingParams(max_tokens=ns.decode_steps + 8, temperature=0.0, ignore_eos=True)
    for _ in range(ns.concurrency):
        eng.add_request(torch.randint(0, cfg.vocab_size, (ns.isl,), generator=g).tolist(), sp)
    while eng.scheduler.waiting or eng.scheduler.prefilling:
        eng.step()
    for _ in range(ns.decode_steps):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    eng.close()
    print("ok")


if __name__ == "__main__":
    main()
