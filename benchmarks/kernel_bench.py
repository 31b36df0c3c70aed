#!/usr/bin/env python
"""Per-kernel timing of the decode step's ops at the flagship shapes (dense 27B NVFP4, fp8 KV).

Every op is timed with CUDA events after warm-up; weight operands rotate through several
copies so each timed launch streams its weights from HBM (inputs larger than L2), and the
figures are reported against the measured copy bandwidth and cuBLAS bf16 throughput in
MEASURED_PEAKS.json ("of measured") or the fallback peaks ("of fallback").

    python benchmarks/kernel_bench.py [--m 1,16,128] [--ctx 640] [--tp 8] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from metrale_inference_alpha_b200 import ops  # noqa: E402
from metrale_inference_alpha_b200.ops import reference as ref  # noqa: E402

DEV = "cuda"


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


def timeit(fn, iters=20, warmup=3, reps=5):
    """Median device time of one call of fn(i): `iters` calls are captured into one CUDA graph
    (so host launch overhead does not gate small kernels) and the graph is replayed `reps`
    times between CUDA events."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / iters)
    ts.sort()
    return ts[len(ts) // 2] * 1e-3


def rand_weight(N, K, fmt, copies):
    out = []
    for c in range(copies):
        if fmt == "nvfp4":
            w = ops.QuantWeight("nvfp4", N, K, torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=DEV),
                                torch.randint(40, 60, (N, K // 16), dtype=torch.uint8, device=DEV), 1e-3)
            w.prepare_cuda()
        elif fmt == "bf16":
            w = ops.QuantWeight("bf16", N, K, (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16))
        elif fmt == "fp8_row":
            w = ops.QuantWeight("fp8_row", N, K, torch.randint(0, 120, (N, K), dtype=torch.uint8, device=DEV),
                                torch.rand(N, device=DEV) * 0.01)
        else:
            w = ops.QuantWeight("fp8_block", N, K, torch.randint(0, 120, (N, K), dtype=torch.uint8, device=DEV),
                                torch.rand((N + 127) // 128, (K + 127) // 128, device=DEV) * 0.01)
        out.append(w)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", default="1,16,128")
    ap.add_argument("--ctx", type=int, default=640)
    ap.add_argument("--fmt", default="nvfp4")
    ap.add_argument("--json", default="")
    ap.add_argument("--splits", default="")
    ap.add_argument("--tp", type=int, default=1, help="time one rank's share of the shapes under N-way tensor parallelism")
    args = ap.parse_args()
    hbm, tflops, tag = peaks()
    H, I, V, Hq, Hkv, D = 5120, 17408 // args.tp, (151936 + args.tp - 1) // args.tp, 40 // args.tp, max(1, 8 // args.tp), 128
    rows = []
    fmt = args.fmt
    afmt = ops.ACT_FOR_WEIGHT[fmt]
    wbytes = {"nvfp4": 0.5 + 1 / 16, "bf16": 2.0, "fp8_row": 1.0, "fp8_block": 1.0}[fmt]

    def report(name, M, sec, nbytes, flops=0.0):
        gbs = nbytes / sec / 1e9
        tf = flops / sec / 1e12
        rows.append(dict(op=name, M=M, us=round(sec * 1e6, 2), GBs=round(gbs, 1), frac_hbm=round(gbs / hbm, 3),
                         TFLOPs=round(tf, 1), frac_tensor=round(tf / tflops, 3)))
        print(f"{name:28s} M={M:4d} {sec*1e6:9.2f} us  {gbs:8.1f} GB/s ({gbs/hbm:5.1%} {tag})  "
              f"{tf:7.1f} TFLOP/s ({tf/tflops:5.1%} {tag})", flush=True)

    gemms = [("qkv", (Hq + 2 * Hkv) * D, H, False), ("o_proj", H, Hq * D, False), ("gate_up+swiglu", 2 * I, H, True),
             ("down", H, I, False)]
    for M in [int(x) for x in args.m.split(",")]:
        x = torch.randn(M, H, device=DEV).to(torch.bfloat16)
        # norm + quant
        w_ln = torch.ones(H, device=DEV, dtype=torch.bfloat16)
        t = timeit(lambda i: ops.row_op(x, afmt, ops.IN_RMSNORM, w=w_ln))
        report(f"rmsnorm+quant[{afmt}]", M, t, M * H * 2.6)
        for name, N, K, sw in gemms:
            copies = max(2, int(400e6 // (N * K * wbytes)) + 1)
            ws = rand_weight(N, K, fmt, copies)
            act = ops.quantize_act(torch.randn(M, K, device=DEV).to(torch.bfloat16), afmt)
            out = torch.empty(M, N // 2 if sw else N, device=DEV, dtype=torch.bfloat16)
            t = timeit(lambda i: ops.linear(act, ws[i % copies], swiglu=sw, out=out))
            report(f"gemm {name} [{fmt}]", M, t, N * K * wbytes + M * K * wbytes + M * N * 2, 2.0 * M * N * K)
            del ws
        # lm_head bf16
        ws = rand_weight(V, H, "bf16", 2)
        act = ops.quantize_act(x, "bf16")
        out = torch.empty(M, V, device=DEV, dtype=torch.bfloat16)
        t = timeit(lambda i: ops.linear(act, ws[i % 2], out=out), iters=6)
        report("gemm lm_head [bf16]", M, t, V * H * 2 + M * V * 2, 2.0 * M * V * H)
        t = timeit(lambda i: ops.argmax(out))
        report("argmax", M, t, M * V * 2)
        del ws
        # attention: M sequences at ctx tokens, fp8 KV
        ctx, bs = args.ctx, 16
        nblk = (ctx + bs - 1) // bs
        nb = M * nblk + 1
        kc = torch.randint(0, 100, (nb, bs, Hkv, D), dtype=torch.uint8, device=DEV)
        vc = torch.randint(0, 100, (nb, bs, Hkv, D), dtype=torch.uint8, device=DEV)
        bt = (torch.arange(M * nblk, device=DEV, dtype=torch.int32) + 1).view(M, nblk)
        bt_full = torch.zeros(M, 128, dtype=torch.int32, device=DEV)
        bt_full[:, :nblk] = bt
        q = torch.randn(M, Hq, D, device=DEV).to(torch.bfloat16)
        qs = torch.arange(M, device=DEV, dtype=torch.int32)
        ql = torch.ones(M, device=DEV, dtype=torch.int32)
        cl = torch.full((M,), ctx, device=DEV, dtype=torch.int32)
        sc = torch.tensor([0.05], device=DEV)
        t = timeit(lambda i: ops.paged_attention(q, kc, vc, bt_full, qs, ql, cl, max_q_len=1, max_ctx=2048,
                                                 scale=1 / math.sqrt(D), k_scale=sc, v_scale=sc))
        report(f"paged_attn fp8 ctx={ctx}", M, t, 2.0 * M * ctx * Hkv * D)
        qkv = torch.randn(M, (Hq + 2 * Hkv) * D, device=DEV).to(torch.bfloat16)
        pos = torch.full((M,), ctx - 1, device=DEV, dtype=torch.int32)
        slots = (bt[:, -1].long() * bs + (ctx - 1) % bs)
        cos, sin = ref.rope_tables(2048, D, 1e6, device=DEV)
        nw = torch.ones(D, device=DEV, dtype=torch.bfloat16)
        t = timeit(lambda i: ops.qk_norm_rope_kvwrite(qkv, Hq=Hq, Hkv=Hkv, D=D, positions=pos, slots=slots,
                                                      k_cache=kc, v_cache=vc, q_norm_w=nw, k_norm_w=nw, cos=cos,
                                                      sin=sin, k_scale=sc, v_scale=sc))
        report("qk_norm+rope+kvwrite", M, t, M * (Hq + 2 * Hkv) * D * 2 * 2)
        a16 = torch.randn(M, I, device=DEV).to(torch.bfloat16)
        t = timeit(lambda i: ops.quantize_act(a16, afmt))
        report(f"quant act[{afmt}] K={I}", M, t, M * I * 2.6)
    if args.json:
        json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "tag": tag}, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
