#!/usr/bin/env python
"""Timing of the kernels outside the five headline configurations: Kimi delta attention, the
sparse-attention indexer / top-k / gather, the hyper-connection highway ops and the storage tier's tiled
attention. CUDA events after warm-up, several launches captured in one graph, inputs rotated through
copies larger than L2 where the op is bandwidth-bound; figures against the measured copy bandwidth
("of measured") or the fallback peak.

    python benchmarks/ext_bench.py [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kernel_bench import peaks, timeit  # noqa: E402
from metrale_inference_alpha_b200.engine.batch import ForwardBatch  # noqa: E402
from metrale_inference_alpha_b200.ops import highway as hw  # noqa: E402
from metrale_inference_alpha_b200.ops import recurrent as rops  # noqa: E402
from metrale_inference_alpha_b200.ops import sparse_attn as SA  # noqa: E402
from metrale_inference_alpha_b200.storage import kernels as SK  # noqa: E402

DEV = "cuda"


def _batch(lens, start=0):
    nb = (max(lens) + start) // 16 + 1
    seqs = [dict(tokens=[1] * n, start_pos=start, blocks=list(range(1, nb + 1)), state_slot=i + 1) for i, n in enumerate(lens)]
    return ForwardBatch.build(seqs, 16, device=DEV)


def kda(rows):
    H, D = 32, 128
    for name, lens, start in (("decode, 128 sequences", [1] * 128, 5), ("prefill, 1 x 4096 tokens", [4096], 0)):
        T = sum(lens)
        g = torch.Generator(device=DEV).manual_seed(0)
        conv = torch.randn(T, 3 * H * D, device=DEV, generator=g)
        g_raw, b_raw = torch.randn(T, H * D, device=DEV, generator=g), torch.randn(T, H, device=DEV, generator=g)
        A, dtb = torch.zeros(H, device=DEV), torch.zeros(H * D, device=DEV)
        st = torch.zeros(len(lens) + 1, H, D, D, device=DEV)
        gate = torch.randn(T, H * D, device=DEV, generator=g).to(torch.bfloat16)
        w = torch.ones(D, device=DEV)
        b = _batch(lens, start)
        t = timeit(lambda i: rops.kda_recurrence(conv, g_raw, b_raw, A, dtb, -5.0, st, b, heads=H, dim=D, norm=(w, gate, 1e-6)),
                   iters=4 if T > 1000 else 20)
        byt = (conv.numel() + g_raw.numel()) * 4 + gate.numel() * 2 + T * H * D * 2 + (2 * len(lens) * H * D * D * 4)
        rows.append({"op": f"kda_recurrence ({name}, 32 heads x 128)", "us": t * 1e6, "gbs": byt / t / 1e9})


def sparse(rows):
    Hi, Di, bs, ctx, k = 64, 128, 16, 32768, 2048
    nb = ctx // bs + 2
    g = torch.Generator(device=DEV).manual_seed(1)
    for T in (1, 16):
        kc = torch.randn(nb * T, bs, 1, Di, device=DEV, generator=g).to(torch.bfloat16)
        table = (torch.arange(T, device=DEV, dtype=torch.int32)[:, None] * nb + torch.arange(nb, device=DEV, dtype=torch.int32)[None, :] ) % (nb * T)
        row_seq = torch.arange(T, device=DEV, dtype=torch.int32)
        row_ctx = torch.full((T,), ctx, device=DEV, dtype=torch.int32)
        iq = torch.randn(T, Hi, Di, device=DEV, generator=g).to(torch.bfloat16)
        iw = torch.rand(T, Hi, device=DEV, generator=g)
        t = timeit(lambda i: SA.index_scores(iq, iw, kc, table, row_seq, row_ctx, ctx), iters=5)
        rows.append({"op": f"index_score ({T} rows x ctx {ctx}, 64 x 128 indexer)", "us": t * 1e6,
                     "gbs": T * ctx * Di * 2 / t / 1e9, "tflops": 2.0 * T * ctx * Hi * Di / t / 1e12})
        sc = SA.index_scores(iq, iw, kc, table, row_seq, row_ctx, ctx)
        t = timeit(lambda i: SA.topk_indices(sc, row_ctx, k), iters=5)
        rows.append({"op": f"topk_select ({T} rows, {k} of {ctx})", "us": t * 1e6, "gbs": 5 * T * ctx * 4 / t / 1e9})
        cache = torch.randn(nb * T, bs, 1, 576, device=DEV, generator=g).to(torch.bfloat16)
        idx, cnt = SA.topk_indices(sc, row_ctx, k)
        t = timeit(lambda i: SA.gather_rows(cache, table, row_seq, idx, cnt), iters=5)
        rows.append({"op": f"gather_rows ({T} rows x {k} x 1152 B)", "us": t * 1e6, "gbs": 2 * T * k * 1152 / t / 1e9})


def highway(rows):
    T, hc, H = 128, 4, 5120
    g = torch.Generator(device=DEV).manual_seed(2)
    streams = torch.randn(T, hc, H, device=DEV, generator=g)
    fn = (torch.randn((2 + hc) * hc, hc * H, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    scale, base = torch.ones(3, device=DEV), torch.zeros((2 + hc) * hc, device=DEV)
    t = timeit(lambda i: hw.hc_pre(streams, fn, scale, base, iters=20))
    rows.append({"op": f"hc_pre ({T} rows, 4 streams x 5120)", "us": t * 1e6, "gbs": (streams.numel() * 4 + T * H * 2) / t / 1e9})
    y, post, comb = hw.hc_pre(streams, fn, scale, base, iters=20)
    t = timeit(lambda i: hw.hc_post(y, streams, post, comb))
    rows.append({"op": f"hc_post ({T} rows, 4 streams x 5120)", "us": t * 1e6, "gbs": (2 * streams.numel() * 4 + T * H * 2) / t / 1e9})


def storage(rows):
    S, Hq, Hkv, D, bs, nblk = 8, 40, 8, 128, 16, 256                    # a tile of 4096 tokens per sequence
    g = torch.Generator(device=DEV).manual_seed(3)
    for fp8 in (False, True):
        k = torch.randn(S * nblk, bs, Hkv, D, device=DEV, generator=g)
        v = torch.randn(S * nblk, bs, Hkv, D, device=DEV, generator=g)
        pk, pv = ((k.to(torch.float8_e4m3fn).view(torch.uint8), v.to(torch.float8_e4m3fn).view(torch.uint8)) if fp8
                  else (k.to(torch.bfloat16), v.to(torch.bfloat16)))
        q = torch.randn(S, Hq, D, device=DEV, generator=g).to(torch.bfloat16)
        tb = torch.arange(S * nblk, device=DEV, dtype=torch.int32).view(S, nblk)
        tc = torch.full((S,), nblk, device=DEV, dtype=torch.int32)
        st = SK.attn_state(S, Hq, D, DEV)
        t = timeit(lambda i: SK.kv_tile_attn(q, pk, pv, tb, tc, st, Hkv=Hkv, block_size=bs, strides=SK.paged_strides(bs, Hkv, D)), iters=5)
        byt = 2 * S * nblk * bs * Hkv * D * (1 if fp8 else 2)
        rows.append({"op": f"kv_tile_attn (8 seqs x 4096 tokens, 40 / 8 heads, {'e4m3' if fp8 else 'bf16'})", "us": t * 1e6, "gbs": byt / t / 1e9})


def moe_nvfp4(rows):
    """Routed NVFP4 (W4A4) experts of a 128-expert, top-8 block (hidden 2048, expert width 768): the grouped
    tcgen05 GEMM over 128-row aligned expert segments against one GEMM per active expert."""
    from types import SimpleNamespace

    from kernel_bench import rand_weight
    from metrale_inference_alpha_b200 import ops
    from metrale_inference_alpha_b200.models.decoder import Decoder
    from metrale_inference_alpha_b200.models.moe import routed_experts
    from metrale_inference_alpha_b200.ops.moe import stack_experts
    from metrale_inference_alpha_b200.weights.loader import FfnW, MoeW
    E, K, H, I = 128, 8, 2048, 768
    experts = [FfnW(rand_weight(2 * I, H, "nvfp4", 1)[0], rand_weight(H, I, "nvfp4", 1)[0], interleaved=True) for _ in range(E)]
    w = MoeW(experts=experts, expert_lo=0)
    w.grouped = stack_experts(experts)
    cfg = SimpleNamespace(experts_per_token=K, ffn_act="swiglu", hidden_size=H, num_experts=E)
    dec = SimpleNamespace(cfg=cfg, _as_act=Decoder._as_act)
    g = torch.Generator(device=DEV).manual_seed(5)
    wbytes = sum(e.gate_up.nbytes() + e.down.nbytes() for e in experts) / E
    for T in (64, 2048):
        x = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
        a = ops.row_op(x, "nvfp4", also_bf16=True)[0]
        idx = torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(T)]).to(torch.int32)
        wts = torch.rand(T, K, device=DEV, generator=g)
        active = int(idx.unique().numel())
        flops = 2.0 * T * K * (2 * I * H + H * I)
        t_g = timeit(lambda i: routed_experts(dec, a, wts, idx, w), iters=10)
        grouped, w.grouped = w.grouped, None
        try:
            for _ in range(2):
                routed_experts(dec, a, wts, idx, w)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                routed_experts(dec, a, wts, idx, w)
            e1.record()
            torch.cuda.synchronize()
            t_e = e0.elapsed_time(e1) / 3 * 1e-3
        finally:
            w.grouped = grouped
        for name, t in (("grouped GEMM, graph replay", t_g), ("one GEMM per active expert, eager", t_e)):
            rows.append({"op": f"nvfp4 experts ({T} tokens x top-8 of 128, {active} active; {name})", "us": t * 1e6,
                         "gbs": active * wbytes / t / 1e9, "tflops": flops / t / 1e12})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None, help="run one section: kda | sparse | highway | storage | moe_nvfp4")
    ns = ap.parse_args()
    hbm, _, tag = peaks()
    rows = []
    for f in (kda, sparse, highway, storage, moe_nvfp4):
        if ns.only in (None, f.__name__):
            f(rows)
    for r in rows:
        r["frac_hbm"] = r["gbs"] / hbm
        extra = f", {r['tflops']:.1f} TFLOP/s" if "tflops" in r else ""
        print(f"{r['op']:<72} {r['us']:>10.1f} us  {r['gbs']:>8.1f} GB/s = {r['frac_hbm']:.1%} {tag}{extra}")
    if ns.json:
        json.dump({"peaks": tag, "rows": rows}, open(ns.json, "w"), indent=1)


if __name__ == "__main__":
    main()
