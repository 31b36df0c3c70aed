#!/usr/bin/env python
"""Runs one op a few times, eagerly, at the flagship decode shape: the target of
`ncu --set full -k regex:<kernel> -c 3` captures (small case: a few hundred MB on the device).

    python benchmarks/ncu_case.py --op attn   [--m 128 --ctx 640]
    python benchmarks/ncu_case.py --op gemm   [--m 128 --n 5120 --k 17408 --fmt nvfp4]
    python benchmarks/ncu_case.py --op rowop  [--m 128 --k 5120]
    python benchmarks/ncu_case.py --op mla    [--m 64 --ctx 2048]
    python benchmarks/ncu_case.py --op kda_prefill [--ctx 4096]
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from metrale_inference_alpha_b200 import ops  # noqa: E402
from kernel_bench import rand_weight  # noqa: E402

DEV = "cuda"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="attn")
    ap.add_argument("--m", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=640)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--k", type=int, default=17408)
    ap.add_argument("--fmt", default="nvfp4")
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--swiglu", action="store_true", help="--op gemm: SwiGLU epilogue (gate / up rows interleaved)")
    ap.add_argument("--impl", type=int, default=0, help="--op mla: 1 = mma.sync kernel, 2 = tcgen05 kernel, 0 = the engine's choice")
    ap.add_argument("--ranks", type=int, default=8, help="--op tpfused: emulated ranks (partials summed by one kernel)")
    a = ap.parse_args()
    M = a.m
    if a.op == "attn":
        Hq, Hkv, D, bs = 40, 8, 128, 16
        nblk = (a.ctx + bs - 1) // bs
        nb = M * nblk + 1
        kc = torch.randint(0, 100, (nb, bs, Hkv, D), dtype=torch.uint8, device=DEV)
        vc = torch.randint(0, 100, (nb, bs, Hkv, D), dtype=torch.uint8, device=DEV)
        bt = torch.zeros(M, 128, dtype=torch.int32, device=DEV)
        bt[:, :nblk] = (torch.arange(M * nblk, device=DEV, dtype=torch.int32) + 1).view(M, nblk)
        q = torch.randn(M, Hq, D, device=DEV).to(torch.bfloat16)
        qs = torch.arange(M, device=DEV, dtype=torch.int32)
        ql = torch.ones(M, device=DEV, dtype=torch.int32)
        cl = torch.full((M,), a.ctx, device=DEV, dtype=torch.int32)
        sc = torch.tensor([0.05], device=DEV)
        for _ in range(a.iters):
            ops.paged_attention(q, kc, vc, bt, qs, ql, cl, max_q_len=1, max_ctx=2048, scale=1 / math.sqrt(D),
                                k_scale=sc, v_scale=sc)
    elif a.op == "prefill_attn":
        # one sequence of --ctx query tokens over its own keys (fresh prefill), 40 / 8 heads of 128, e4m3 cache:
        # the tcgen05 / TMEM kernel (csrc/attention_tc.cu); --fmt bf16 for a bf16 cache
        Hq, Hkv, D, bs, q = 40, 8, 128, 16, a.ctx
        nblk = (q + bs - 1) // bs
        if a.fmt == "bf16":
            kc = torch.randn(nblk + 1, bs, Hkv, D, device=DEV).to(torch.bfloat16)
            vc = torch.randn(nblk + 1, bs, Hkv, D, device=DEV).to(torch.bfloat16)
            sc = None
        else:
            kc = torch.randint(32, 100, (nblk + 1, bs, Hkv, D), dtype=torch.uint8, device=DEV)
            vc = torch.randint(32, 100, (nblk + 1, bs, Hkv, D), dtype=torch.uint8, device=DEV)
            sc = torch.tensor([0.05], device=DEV)
        bt = (torch.arange(nblk, device=DEV, dtype=torch.int32) + 1).view(1, nblk).contiguous()
        qq = torch.randn(q, Hq, D, device=DEV).to(torch.bfloat16)
        ql = torch.tensor([q], dtype=torch.int32, device=DEV)
        qs = torch.zeros(1, dtype=torch.int32, device=DEV)
        for _ in range(a.iters):
            ops.paged_attention(qq, kc, vc, bt, qs, ql, ql, max_q_len=q, max_ctx=q, scale=1 / math.sqrt(D),
                                k_scale=sc, v_scale=sc, force_mode=3)
    elif a.op == "mla":
        # absorbed MLA decode: 128 heads of 576-wide latent queries against a [blocks, 16, 1, 576] latent cache
        from metrale_inference_alpha_b200.ops import mla_cuda
        H, ROW, bs = 128, 576, 16
        nblk = (a.ctx + bs - 1) // bs
        cache = (torch.randn(M * nblk + 1, bs, 1, ROW, device=DEV) * 0.3).to(torch.bfloat16)
        bt = torch.zeros(M, max(nblk, 128), dtype=torch.int32, device=DEV)
        bt[:, :nblk] = (torch.arange(M * nblk, device=DEV, dtype=torch.int32) + 1).view(M, nblk)
        q = (torch.randn(M, H, ROW, device=DEV) * 0.3).to(torch.bfloat16)
        qs = torch.arange(M, device=DEV, dtype=torch.int32)
        ql = torch.ones(M, device=DEV, dtype=torch.int32)
        cl = torch.full((M,), a.ctx, device=DEV, dtype=torch.int32)
        for _ in range(a.iters):
            mla_cuda.mla_attention(q, cache, bt, qs, ql, cl, max_q_len=1, max_ctx=max(nblk, 128) * bs, scale=1 / math.sqrt(192), impl=a.impl)
    elif a.op == "gemm":
        ws = rand_weight(a.n, a.k, a.fmt, 3)
        act = ops.quantize_act(torch.randn(M, a.k, device=DEV).to(torch.bfloat16), ops.ACT_FOR_WEIGHT[a.fmt])
        out = torch.empty(M, a.n // 2 if a.swiglu else a.n, device=DEV, dtype=torch.bfloat16)
        for i in range(a.iters):
            ops.linear(act, ws[i % 3], out=out, swiglu=a.swiglu)
    elif a.op == "tpfused":
        # the consumer-fused tensor-parallel reduction with the ranks emulated on one GPU: one launch sums
        # `ranks` local partial buffers through the peer-load path, adds the residual, normalises, quantises
        from metrale_inference_alpha_b200.parallel.fused import FusedReduce, PendingSum
        fr = FusedReduce(0, 1, DEV, a.n, max(M, 16), emulate=a.ranks)
        w = torch.ones(a.n, device=DEV, dtype=torch.bfloat16)
        res = torch.randn(M, a.n, device=DEV).to(torch.bfloat16)
        for i in range(a.iters):
            for r in range(a.ranks):
                fr.partial_view(M, r).normal_()
            pend = PendingSum(fr, fr.partial_view(M, 0), res)
            fr.reduce_norm(pend, w, "nvfp4", eps=1e-6)
    elif a.op == "kda_prefill":
        # one sequence of --ctx tokens through the chunked Kimi-delta-attention kernels, 32 heads x 128
        # (workspace 70 KB per chunk and head: 0.3 GB at 4096 tokens)
        from metrale_inference_alpha_b200.engine.batch import ForwardBatch
        from metrale_inference_alpha_b200.ops import recurrent as rops
        H, D, T = 32, 128, a.ctx
        conv = torch.randn(T, 3 * H * D, device=DEV)
        g_raw, b_raw = torch.randn(T, H * D, device=DEV), torch.randn(T, H, device=DEV)
        A, dtb = torch.zeros(H, device=DEV), torch.zeros(H * D, device=DEV)
        st = torch.zeros(2, H, D, D, device=DEV)
        gate = torch.randn(T, H * D, device=DEV).to(torch.bfloat16)
        wn = torch.ones(D, device=DEV)
        b = ForwardBatch.build([dict(tokens=[1] * T, start_pos=0, blocks=list(range(1, T // 16 + 2)), state_slot=1)], 16, device=DEV)
        for _ in range(a.iters):
            rops.kda_recurrence(conv, g_raw, b_raw, A, dtb, -5.0, st, b, heads=H, dim=D, norm=(wn, gate, 1e-6))
    elif a.op == "rowop":
        x = torch.randn(M, a.k, device=DEV).to(torch.bfloat16)
        w = torch.ones(a.k, device=DEV, dtype=torch.bfloat16)
        for _ in range(a.iters):
            ops.row_op(x, ops.ACT_FOR_WEIGHT[a.fmt], ops.IN_RMSNORM, w=w)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    print("ok")


if __name__ == "__main__":
    main()
