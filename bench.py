#!/usr/bin/env python
"""Headline benchmark: aggregate decode tokens/s of the dense ~27B NVFP4 model (fp8 KV) on the
reference's ISL128 / OSL1024 concurrency ladder, on N GPUs of one node. N > 1 shards ONE engine
over the N GPUs with tensor parallelism (the configuration's TP = 1/2/4/8 sweep; C requests in
total, strong scaling): row-parallel GEMMs leave their partial sums in NVLink peer memory and
the all-reduce runs inside the RMSNorm + quantiser kernel that consumes it (`--no-fused`: NCCL
all-reduce after the GEMM, the reference's scheme). `--parallelism dp` runs one replica per GPU
instead (weak scaling).

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 64 --warmup 8

Workload (reference ladder semantics): C requests arrive at once, prompts are 128 uniform
random token ids (seed 42), temperature 0, context 2048, batch cap 128, OSL 1024, EOS ignored.
Weights are random N(0, 0.02) quantised to NVFP4 (e2m1 + per-16 e4m3 scales + fp32 global
scale), bf16 embeddings / lm_head; there is no network for a real checkpoint.

What is measured (all as the max over ranks; rank 0 prints ONE JSON line):
  value    K decode steps at concurrency C around the middle of the generation (context ~640,
           reached by untimed fast-forward steps), replayed as CUDA graphs from device-resident
           metadata and timed with CUDA events: the kernel-only view of a step.
  e2e      the ladder rung itself through the public API (`LLMEngine.add_request` / `step`):
           C requests arrive at once, every one generates OSL tokens; value = sum of completion
           tokens / wall time of the batch, prefill included; p50 TTFT from the same run. Every
           step stages its metadata in pinned host memory, copies it host -> device, and reads
           the sampled ids (and the kernels' status word) device -> host. `e2e.k_steps` is the
           same K steps as `value`, driven through `step()`.
  config.ladder   the same end-to-end measurement for every rung 1..128 (`--no-ladder` skips it).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

BASELINE_TOKS = {1: 23.59, 2: 41.02, 4: 74.21, 8: 125.95, 16: 203.36, 32: 291.01, 64: 386.63, 128: 478.11}
# published GB10 ladders of the other configurations' closest reference models (tok/s by concurrency)
BASELINE_OTHER = {"qwen-hybrid-moe-35b-fp8": {1: 84.99, 2: 127.12, 4: 180.24, 8: 235.82, 16: 311.18}}
WEIGHT_DESC = {"nvfp4": "nvfp4 weights x nvfp4 activations (fp32 accumulate)", "fp8_block": "fp8 e4m3 128x128-block weights x fp8 activations",
               "fp8_row": "fp8 e4m3 per-row weights x fp8 activations", "bf16": "bf16"}
SMI_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def reference_arm(args) -> int:
    """The reference is a Rust workspace (no setup.py / pyproject, needs cargo + crates.io +
    CUDA 13.0): an offline `pip install --no-index --target baseline/_ref <reference checkout>`
    reports "not installable"."""
    line = {"impl": "reference",
            "unavailable": "reference is a Cargo workspace (Rust 1.93.1 + CUDA 13.0 + ~400 crates); "
                           "pip reports 'neither setup.py nor pyproject.toml found'; no cargo/rustc offline"}
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(line), flush=True)
    return 0


class ClockSampler:
    def __init__(self, gpu_index: int):
        self.proc = None
        self.path = f"/tmp/bench_clocks_{os.getpid()}.csv"
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2])); power.append(float(p[3]))
            except ValueError:
                continue
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm), power_w_max=max(power))
        return out


def torch_arm(args, cfg, rank: int, world: int, local: int, dev: str) -> int:
    """`--impl torch`: K graph-replayed decode steps of the same shape, batch and context from
    library kernels only (bf16 weights: cuBLAS has no NVFP4 x NVFP4 path here)."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from benchmarks.torch_baseline import run as torch_run
    C = args.concurrency
    ctx = args.isl + args.osl // 2
    sampler = ClockSampler(local)
    sampler.start()
    r = torch_run(cfg, C, ctx, args.steps, args.warmup, rank, world, dev)
    clocks = sampler.stop()
    line = {"metric": "aggregate decode tok/s at C=%d (ISL128/OSL1024), dense 27B, library kernels" % C,
            "value": round(r["tok_s"], 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(r["ms_per_step"], 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(r["tok_s"] / BASELINE_TOKS.get(C, BASELINE_TOKS[128]), 3),
            "dtype": "bf16 weights and activations (cuBLAS), bf16 KV (SDPA)", "data": "synthetic: random-init bf16 weights",
            "config": {"model": cfg.name, "layers": cfg.num_layers, "hidden": cfg.hidden_size, "global_batch": C,
                       "seq_len": args.isl, "osl": args.osl, "ctx_in_timed_window": ctx, "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2 (weights %.1f GB per GPU)" % (r["weight_bytes"] / 1e9),
                       "value_is": "K graph-replayed decode steps at C, CUDA events, max over ranks"},
            "e2e": None, "gpu_launches": 0, "clocks": clocks, "impl": "torch"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"],
                    help="reference: the reference engine (does not build offline: prints `unavailable`); torch: the "
                         "same step from PyTorch's library kernels (cuBLAS bf16, SDPA, NCCL), see benchmarks/torch_baseline.py")
    ap.add_argument("--concurrency", type=int, default=128)
    ap.add_argument("--model", default="dense-27b-nvfp4")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (marks the line invalid)")
    ap.add_argument("--isl", type=int, default=128)
    ap.add_argument("--osl", type=int, default=1024)
    ap.add_argument("--no-fast-forward", action="store_true")
    ap.add_argument("--fused", action="store_true", help="accepted for compatibility: the fused reduction is the default")
    ap.add_argument("--no-fused", action="store_true",
                    help="tensor parallel: NCCL all-reduce after the row-parallel GEMMs + separate norm kernel "
                         "(the reference's scheme) instead of the reduction fused into its consumer")
    ap.add_argument("--no-ladder", action="store_true", help="skip the full-OSL ladder (e2e then covers rung C only)")
    ap.add_argument("--ladder", action="store_true", help="accepted for compatibility: the ladder runs by default")
    ap.add_argument("--rungs", default="1,2,4,8,16,32,64,128")
    ap.add_argument("--ttft-reps", type=int, default=0,
                    help="also measure p50 time to first token of single requests of --isl tokens, cold and prefix-warm")
    ap.add_argument("--ep-dispatch", default="allreduce", choices=["allreduce", "a2a"],
                    help="--parallelism ep: masked-local experts + all-reduce, or token dispatch over NVLink peer memory")
    ap.add_argument("--speculative", default="off", choices=["off", "mtp"],
                    help="mtp: after the headline run, also report what a verify step (K = 1..4) and the "
                         "draft proposal cost next to a decode step at C = 8 (1 GPU; benchmarks/spec_cost.py)")
    ap.add_argument("--parallelism", default="tp", choices=["dp", "tp", "ep"],
                    help="N>1: tp = one engine sharded over N GPUs, C requests in total (strong scaling, the "
                         "configuration's TP sweep); dp = one engine replica per GPU, each serving C requests")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    tp = None
    use_ep = world > 1 and args.parallelism == "ep"        # attention tensor-parallel, experts expert-parallel
    use_tp = world > 1 and args.parallelism in ("tp", "ep")
    replicas = world if not use_tp else 1
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(dev))
        if use_tp:
            from metrale_inference_alpha_b200.parallel.tp import NcclTpContext
            tp = NcclTpContext(rank, world, dev, fused=not args.no_fused)
            if use_ep:
                tp.ep_rank = rank

    from metrale_inference_alpha_b200.config.model_config import preset
    if args.impl == "torch":
        return torch_arm(args, preset(args.model), rank, world, local, dev)
    from metrale_inference_alpha_b200 import ops
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams

    cfg = preset(args.model)
    if args.layers:
        cfg = cfg.scaled(num_layers=args.layers, layer_types=cfg.layer_types[:args.layers],
                         ffn_types=cfg.ffn_types[:args.layers])
    ctx_len = max(2048, args.isl + args.osl + 16)
    base_toks = BASELINE_TOKS if args.model == "dense-27b-nvfp4" else BASELINE_OTHER.get(args.model, {})

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run_rung(C: int, steps: int, warmup: int, eng=None):
        if eng is None:
            eng = LLMEngine(EngineArgs(model=cfg, device=dev, max_num_seqs=128, max_model_len=ctx_len,
                                       max_prefill_tokens=8192, enable_prefix_caching=True,
                                       gpu_memory_utilization=0.85, tp_size=world if use_tp else 1,
                                       ep_size=world if use_ep else 1, ep_dispatch=args.ep_dispatch, seed=0), tp=tp)
        g = torch.Generator().manual_seed(42 + (0 if use_tp else rank))
        prompts = [torch.randint(0, cfg.vocab_size, (args.isl,), generator=g).tolist() for _ in range(C)]
        sp = SamplingParams(max_tokens=args.osl, temperature=0.0, ignore_eos=True)
        barrier()
        t_arrive = time.perf_counter()
        for p in prompts:
            eng.add_request(p, sp)
        ttfts = {}
        while eng.scheduler.waiting or eng.scheduler.prefilling:
            for o in eng.step():
                if o.ttft_ms is not None and o.request_id not in ttfts:
                    ttfts[o.request_id] = (time.perf_counter() - t_arrive) * 1e3
        torch.cuda.synchronize()
        # fast-forward (untimed) so the timed window sits around the middle of the generation
        target_ctx = args.isl + args.osl // 2
        ff = 0 if args.no_fast_forward else max(0, target_ctx - steps - warmup - args.isl - 1)
        ff = min(ff, args.osl - 2 * steps - warmup - 8)
        for _ in range(max(0, ff)):
            eng.step()
        for _ in range(warmup):
            eng.step()
        sampler = ClockSampler(local)
        # ---- e2e: public API ticks, host->device metadata + device->host token ids each step
        barrier()
        h0, d0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes
        sampler.start()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        tokens_before = eng.scheduler.stats["decode_tokens"]
        e0.record()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        barrier()
        e2e_s = max_over_ranks(max(wall, e0.elapsed_time(e1) / 1e3))
        e2e_tokens = eng.scheduler.stats["decode_tokens"] - tokens_before
        h2d = (eng.runner.h2d_bytes - h0) / steps
        d2h = (eng.runner.d2h_bytes - d0) / steps
        # ---- kernel-only: replay the decode graph of this rung from device-resident metadata
        eng.flush()                                       # a step launched ahead is applied first
        plan = eng.scheduler.plan()
        rung = eng.runner._rung(len(plan.items))
        key = (rung, True, False)
        eng.runner._stage(plan, pad_seqs=rung)
        graph = eng.runner.graphs[key][0]
        launches_per_step = eng.runner.graphs[key][1]
        for _ in range(3):
            graph.replay()
        barrier()
        k0 = torch.cuda.Event(enable_timing=True); k1 = torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(steps):
            graph.replay()
        k1.record()
        torch.cuda.synchronize()
        barrier()
        clocks = sampler.stop()
        dev_s = max_over_ranks(k0.elapsed_time(k1) / 1e3)
        # hand the planned step back to the scheduler so its bookkeeping stays consistent
        res = eng.runner.execute(plan)
        eng.scheduler.apply(plan, res)
        ctx_mid = int(sum(len(s.tokens) for s in eng.scheduler.running) / max(1, len(eng.scheduler.running)))
        for s in list(eng.scheduler.running):
            eng.abort(s.req.request_id)
        tt = sorted(ttfts.values())
        return dict(C=C, tok_s=replicas * C * steps / dev_s, ms_per_step=dev_s / steps * 1e3,
                    e2e_tok_s=replicas * e2e_tokens / e2e_s, e2e_ms_per_step=e2e_s / steps * 1e3, h2d=h2d, d2h=d2h,
                    launches=launches_per_step * steps * world, clocks=clocks, ctx=ctx_mid, ff=ff,
                    ttft_p50_ms=tt[len(tt) // 2] if tt else None, eng=eng)

    C = args.concurrency
    r = run_rung(C, args.steps, args.warmup)
    eng = r.pop("eng")

    # ---- the ladder: every rung end to end through the public API, full OSL, prefill included
    from metrale_inference_alpha_b200.bench.ladder import run_rung as ladder_rung
    rungs = [C] if args.no_ladder else sorted({int(x) for x in args.rungs.split(",") if x} | {C})
    ladder = {}
    for c in rungs:
        ladder_rung(eng, c, min(args.isl, 16), 4, seed=7)          # graph capture / allocator warm-up of the rung
        h0, d0, s0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes, eng.step_count
        barrier()
        row = ladder_rung(eng, c, args.isl, args.osl)
        barrier()
        wall = max_over_ranks(row["wall_s"])
        n_steps = max(1, eng.step_count - s0)
        ladder[c] = {"tok_s": round(replicas * row["tokens"] / wall, 2), "ttft_p50_ms": round(max_over_ranks(row["ttft_p50_ms"]), 1),
                     "decode_ms_per_step": round(row["ms_per_step"], 4), "wall_s": round(wall, 3), "steps": n_steps,
                     "completion_tokens": row["tokens"] * replicas,
                     "h2d_bytes_per_step": int((eng.runner.h2d_bytes - h0) / n_steps) * replicas,
                     "d2h_bytes_per_step": int((eng.runner.d2h_bytes - d0) / n_steps) * replicas,
                     "vs_gb10_published": round(replicas * row["tokens"] / wall / base_toks[c], 2) if c in base_toks else None}
    top = ladder[C]
    ttft = None
    if args.ttft_reps > 0:
        # single requests of ISL tokens: cold (new prompt), then the same prompt again (prefix cache warm)
        cold, warm = [], []
        g2 = torch.Generator().manual_seed(4242)
        for _ in range(args.ttft_reps):
            prompt = torch.randint(0, cfg.vocab_size, (args.isl,), generator=g2).tolist()
            for bucket in (cold, warm):
                barrier()
                t0 = time.perf_counter()
                rid = eng.add_request(prompt, SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True))
                first = None
                while eng.has_work():
                    for o in eng.step():
                        if o.request_id == rid and o.new_token_ids and first is None:
                            torch.cuda.synchronize()
                            first = (time.perf_counter() - t0) * 1e3
                bucket.append(max_over_ranks(first if first is not None else float("nan")))
        med = lambda xs: sorted(xs)[len(xs) // 2]
        ttft = {"isl": args.isl, "reps": args.ttft_reps, "cold_p50_ms": round(med(cold), 2), "prefix_warm_p50_ms": round(med(warm), 2)}
    par = f"ep{world}" if use_ep else (f"tp{world}" if (use_tp or world == 1) else f"dp{world}")
    line = {
        "metric": "aggregate decode tok/s at C=%d (ISL%d/OSL%d), %s, %s KV" % (C, args.isl, args.osl, cfg.name, cfg.kv_dtype),
        "value": round(r["tok_s"], 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(r["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "strong" if (use_tp or world == 1) else "weak", "vs_baseline": round(r["tok_s"] / base_toks[C], 3) if C in base_toks else None,
        "dtype": "%s, bf16 lm_head, %s KV" % (WEIGHT_DESC.get(cfg.weight_format, cfg.weight_format), cfg.kv_dtype),
        "data": "synthetic: random-init N(0,0.02) weights in the %s checkpoint layout, uniform-random prompts (seed 42)" % cfg.weight_format,
        "config": {"model": cfg.name, "layers": cfg.num_layers, "hidden": cfg.hidden_size,
                   "global_batch": C * replicas, "per_gpu_batch": C if not use_tp else None, "seq_len": args.isl, "osl": args.osl, "context": ctx_len,
                   "mean_ctx_in_timed_window": r["ctx"], "fast_forward_steps": r["ff"],
                   "parallelism": par, "ep_dispatch": args.ep_dispatch if use_ep else None,
                   "l2": "inputs larger than L2 (weights %.1f GB per GPU + KV per step)" % (eng.weights.nbytes() / 1e9),
                   "fused_collectives": bool(tp is not None and getattr(tp, "reduce", None) is not None),
                   "speculative": "off (MTP gate: random-init drafts never accepted)",
                   "value_is": "K graph-replayed decode steps at C, CUDA events, max over ranks",
                   "ladder": {str(c): v for c, v in ladder.items()}},
        "e2e": {"value": top["tok_s"], "unit": "tokens/s",
                "is": "ladder rung C end to end: C requests at once, OSL tokens each, completion tokens / batch wall, prefill included",
                "steps": top["steps"], "wall_s": top["wall_s"], "ttft_p50_ms": top["ttft_p50_ms"],
                "h2d_bytes_per_step": top["h2d_bytes_per_step"], "d2h_bytes_per_step": top["d2h_bytes_per_step"],
                "k_steps": {"value": round(r["e2e_tok_s"], 2), "ms_per_step": round(r["e2e_ms_per_step"], 4),
                            "h2d_bytes_per_step": int(r["h2d"]) * replicas, "d2h_bytes_per_step": int(r["d2h"]) * replicas}},
        "gpu_launches": int(r["launches"]),
        "clocks": r["clocks"],
        "ttft_p50_ms": top["ttft_p50_ms"],
        "impl": "ours",
    }
    if ttft is not None:
        line["ttft"] = ttft
    if args.speculative == "mtp" and world == 1:
        del eng
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        from benchmarks.spec_cost import run as spec_cost
        line["speculative_cost"] = spec_cost(args.model, dev, 8, steps=32, isl=args.isl, ctx_len=ctx_len)
    if args.layers:
        line["invalid"] = "debug run with fewer layers"
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # NCCL communicators captured into CUDA graphs do not tear down reliably at interpreter
        # exit; every rank has printed / reduced what it needs, so leave without destructors
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
