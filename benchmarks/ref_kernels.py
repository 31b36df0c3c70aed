#!/usr/bin/env python
"""Kernel-level comparison arm: the reference's own CUDA sources (unmodified), compiled for
sm_100a with the flags its B200 target uses, timed next to the in-tree kernels and next to
PyTorch's library kernels on the decode shapes of the dense 27B configuration.

The reference engine itself is a Cargo workspace that does not build offline, but its kernels
are plain ``extern "C" __global__`` functions and its B200 target recompiles the GB10 sources
for ``sm_100a`` (``kernels/b200/HARDWARE.toml``: ``arch = "sm_100a"``, extra flag
``-DMETRALE_NO_WARP_BLOCKSCALE_MMA``; ``kernels/gb10/common/KERNEL.toml``: ``--fmad=false
-DTQ_PLUS_SIGNS``). Two steps:

    python benchmarks/ref_kernels.py --build [--reference-root DIR]     # needs nvcc, no GPU
        compiles the listed sources into cubins under baseline/_ref/kernels/ (git-ignored)
    python benchmarks/ref_kernels.py --run [--json out.json]            # needs a B200
        loads the cubins with the CUDA driver API, checks every kernel against the fp32
        reference on a small shape first (stops at the first wrong answer), then times it.

Launch geometry and argument order follow the comments in the kernel files and the launchers
in ``crates/model-layers/src/layers/ops`` (``norm.rs``, ``prefill_attn_a.rs``); each use below
cites its source. None of these kernels waits on another CTA.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
OUT_DIR = os.path.join(ROOT, "baseline", "_ref", "kernels")

# (cubin name, source under kernels/gb10/common, extra defines)
SOURCES = [
    ("rms_norm", "rms_norm.cu", []),
    ("argmax_bf16", "argmax_bf16.cu", []),
    ("dense_gemv_bf16", "dense_gemv_bf16.cu", []),
    ("dense_gemv_bf16_batchm", "dense_gemv_bf16_batchm.cu", []),
    ("w4a16_gemv", "w4a16_gemv.cu", []),
    ("w4a16_gemm", "w4a16_gemm.cu", []),
    ("paged_decode_attn_fp8_h128", "paged_decode_attn_fp8.cu", ["-DHDIM=128"]),
]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--fmad=false", "-DTQ_PLUS_SIGNS",
         "-DMETRALE_NO_WARP_BLOCKSCALE_MMA", "-cubin"]


def build(reference_root: str) -> int:
    src_dir = os.path.join(reference_root, "kernels", "gb10", "common")
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC") or "nvcc"
    ok = 0
    for name, src, defs in SOURCES:
        out = os.path.join(OUT_DIR, name + ".cubin")
        cmd = [nvcc, *FLAGS, *defs, "-I", src_dir, os.path.join(src_dir, src), "-o", out]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            print(f"[build] {src}: nvcc failed\n{r.stderr[-2000:]}")
            continue
        ok += 1
        print(f"[build] {src} -> {os.path.relpath(out, ROOT)} ({os.path.getsize(out)} bytes)")
    with open(os.path.join(OUT_DIR, "BUILD.json"), "w") as f:
        json.dump({"flags": FLAGS, "sources": [(n, s, d) for n, s, d in SOURCES]}, f, indent=1)
    return 0 if ok == len(SOURCES) else 1


# --------------------------------------------------------------------------------- run
class RefModule:
    """One cubin loaded into torch's context; kernels are launched on torch's current stream."""

    def __init__(self, name: str):
        from cuda.bindings import driver as cu
        self.cu = cu
        path = os.path.join(OUT_DIR, name + ".cubin")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path}: run `python benchmarks/ref_kernels.py --build` first")
        err, self.mod = cu.cuModuleLoadData(open(path, "rb").read())
        if int(err) != 0:
            raise RuntimeError(f"cuModuleLoadData({name}) -> {err}")
        self.fns = {}

    def launch(self, fn: str, grid, block, args, types):
        import torch
        cu = self.cu
        if fn not in self.fns:
            err, f = cu.cuModuleGetFunction(self.mod, fn.encode())
            if int(err) != 0:
                raise RuntimeError(f"cuModuleGetFunction({fn}) -> {err}")
            self.fns[fn] = f
        stream = torch.cuda.current_stream().cuda_stream
        (err,) = cu.cuLaunchKernel(self.fns[fn], grid[0], grid[1], grid[2], block[0], block[1], block[2], 0, stream,
                                   (tuple(args), tuple(types)), 0)
        if int(err) != 0:
            raise RuntimeError(f"cuLaunchKernel({fn}) -> {err}")


P, U32, U64, F32 = C.c_void_p, C.c_uint, C.c_ulonglong, C.c_float


def run(args) -> int:
    import torch
    from benchmarks.kernel_bench import peaks, timeit
    from metrale_inference_alpha_b200 import ops
    from metrale_inference_alpha_b200.ops import reference as ref
    DEV = "cuda"
    torch.zeros(1, device=DEV)                        # torch's primary context becomes current
    hbm, tflops, tag = peaks()
    mods = {n: RefModule(n) for n, _, _ in SOURCES}
    rows = []

    def check(name, got, want, tol):
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        lim = tol * max(1.0, want.float().abs().max().item())
        ok = err <= lim
        print(f"[check] {name}: max err {err:.4g} (limit {lim:.4g}) {'ok' if ok else 'WRONG'}", flush=True)
        if not ok:
            raise SystemExit(f"reference kernel {name} disagrees with the fp32 reference; stopping")

    # ---- reference kernels as callables -------------------------------------------------
    def ref_rms_norm(x, w, out, eps=1e-6):
        # rms_norm.cu:45 (1 + weight scaling); launcher norm.rs: grid [tokens], block [min(hidden, 1024)]
        M, H = x.shape
        mods["rms_norm"].launch("rms_norm", (M, 1, 1), (min(H, 1024), 1, 1),
                                (x.data_ptr(), w.data_ptr(), out.data_ptr(), H, eps), (P, P, P, U32, F32))

    def ref_argmax(logits, out):
        # argmax_bf16.cu:68 argmax_bf16_batch: one block of 1024 threads per row
        M, V = logits.shape
        mods["argmax_bf16"].launch("argmax_bf16_batch", (M, 1, 1), (1024, 1, 1),
                                   (logits.data_ptr(), out.data_ptr(), V, logits.stride(0)), (P, P, U32, U32))

    def ref_dense_gemv(a, w, out):
        # dense_gemv_bf16.cu: grid ceil(N/4), block 256 (M = 1); dense_gemv_bf16_batchm.cu: grid (ceil(N/4), Y),
        # block 256, at most 16 rows per block row
        M, K = a.shape
        N = w.shape[0]
        if M == 1:
            mods["dense_gemv_bf16"].launch("dense_gemv_bf16", ((N + 3) // 4, 1, 1), (256, 1, 1),
                                           (a.data_ptr(), w.data_ptr(), out.data_ptr(), N, K), (P, P, P, U32, U32))
        else:
            y = (M + 15) // 16
            mods["dense_gemv_bf16_batchm"].launch("dense_gemv_bf16_batchm", ((N + 3) // 4, y, 1), (256, 1, 1),
                                                  (a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, out.stride(0)),
                                                  (P, P, P, U32, U32, U32, U32))

    def ref_w4a16(a, packed, scale, scale2, out):
        # w4a16_gemv.cu: M = 1 w4a16_gemv, M <= 8 w4a16_gemv_batch8 (grid ceil(N/4), block 256);
        # w4a16_gemm.cu: 64x64 tiles, grid (ceil(N/64), ceil(M/64)), block 128
        M, K = a.shape
        N = packed.shape[0]
        if M == 1:
            mods["w4a16_gemv"].launch("w4a16_gemv", ((N + 3) // 4, 1, 1), (256, 1, 1),
                                      (a.data_ptr(), packed.data_ptr(), scale.data_ptr(), scale2, out.data_ptr(), N, K),
                                      (P, P, P, F32, P, U32, U32))
        elif M <= 8:
            mods["w4a16_gemv"].launch("w4a16_gemv_batch8", ((N + 3) // 4, 1, 1), (256, 1, 1),
                                      (a.data_ptr(), packed.data_ptr(), scale.data_ptr(), scale2, out.data_ptr(), M, N, K),
                                      (P, P, P, F32, P, U32, U32, U32))
        else:
            mods["w4a16_gemm"].launch("w4a16_gemm", ((N + 63) // 64, (M + 63) // 64, 1), (128, 1, 1),
                                      (a.data_ptr(), packed.data_ptr(), scale.data_ptr(), scale2, out.data_ptr(), M, N, K),
                                      (P, P, P, F32, P, U32, U32, U32))

    def ref_decode_attn(q, kc, vc, out, bt, seq_lens, k_scale, v_scale):
        # paged_decode_attn_fp8.cu:58 / prefill_attn_a.rs:346: grid (q heads, seqs), block 256
        S, Hq, D = q.shape
        nb, bs, Hkv, _ = kc.shape
        mods["paged_decode_attn_fp8_h128"].launch(
            "paged_decode_attn_fp8", (Hq, S, 1), (256, 1, 1),
            (q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), bt.data_ptr(), seq_lens.data_ptr(), bt.stride(0),
             Hq, Hkv, D, bs, 1.0 / math.sqrt(D), k_scale, v_scale, Hq * D, bs * Hkv * D, 0),
            (P, P, P, P, P, P, U32, U32, U32, U32, U32, F32, F32, F32, U32, U64, U32))

    # ---- correctness on small shapes (stop at the first wrong answer) ---------------------
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 512, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(512, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    out = torch.empty_like(x)
    ref_rms_norm(x, w, out)
    check("rms_norm", out, ref.rms_norm(x.float().cpu(), w.float().cpu(), 1e-6, True).to(DEV), 2e-2)
    lg = torch.randn(5, 4096, generator=g).to(torch.bfloat16).to(DEV)
    ids = torch.zeros(5, dtype=torch.int32, device=DEV)
    ref_argmax(lg, ids)
    check("argmax_bf16_batch", ids, lg.float().argmax(-1), 0)
    for M in (1, 7):
        a = torch.randn(M, 256, generator=g).to(torch.bfloat16).to(DEV)
        wd = (torch.randn(64, 256, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
        o = torch.empty(M, 64, dtype=torch.bfloat16, device=DEV)
        ref_dense_gemv(a, wd, o)
        check(f"dense_gemv_bf16 M={M}", o, a.float() @ wd.float().t(), 2e-2)
    for M in (1, 5, 70):
        qw = ops.make_weight(torch.randn(128, 512, generator=g) * 0.05, "nvfp4")
        a = torch.randn(M, 512, generator=g).to(torch.bfloat16).to(DEV)
        o = torch.empty(M, 128, dtype=torch.bfloat16, device=DEV)
        ref_w4a16(a, qw.data.to(DEV), qw.scale.to(DEV), float(qw.gscale), o)
        check(f"w4a16 M={M}", o, a.float() @ qw.dequant().t().to(DEV), 2e-2)
    S, Hq, Hkv, D, bs, ctx = 3, 8, 2, 128, 16, 50
    nblk = (ctx + bs - 1) // bs
    kc = torch.randint(0x20, 0x48, (S * nblk + 1, bs, Hkv, D), generator=g, dtype=torch.uint8).to(DEV)
    vc = torch.randint(0x20, 0x48, (S * nblk + 1, bs, Hkv, D), generator=g, dtype=torch.uint8).to(DEV)
    bt = (torch.arange(S * nblk, dtype=torch.int32) + 1).view(S, nblk).to(DEV)
    q = torch.randn(S, Hq, D, generator=g).to(torch.bfloat16).to(DEV)
    sl = torch.tensor([50, 33, 17], dtype=torch.int32, device=DEV)
    o = torch.zeros_like(q)
    ref_decode_attn(q, kc, vc, o, bt, sl, 0.05, 0.03)
    one = torch.ones(S, dtype=torch.int32)
    want = ref.paged_attention(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), torch.arange(S, dtype=torch.int32), one, sl.cpu(),
                               1.0 / math.sqrt(D), torch.tensor([0.05]), torch.tensor([0.03]), 0)
    check("paged_decode_attn_fp8", o, want.to(DEV), 2e-2)

    # ---- timings on the decode shapes of the dense 27B configuration ----------------------
    H, I, V, Hq, Hkv, D = 5120, 17408, 151936, 40, 8, 128

    def report(op, impl, M, sec, nbytes):
        gbs = nbytes / sec / 1e9
        rows.append(dict(op=op, impl=impl, M=M, us=round(sec * 1e6, 2), GBs=round(gbs, 1), frac_hbm=round(gbs / hbm, 3)))
        print(f"{op:26s} {impl:10s} M={M:4d} {sec * 1e6:9.2f} us  {gbs:8.1f} GB/s ({gbs / hbm:5.1%} {tag})", flush=True)

    for M in [int(v) for v in args.m.split(",")]:
        x = torch.randn(M, H, device=DEV).to(torch.bfloat16)
        w_ln = torch.zeros(H, device=DEV, dtype=torch.bfloat16)
        o = torch.empty_like(x)
        report("rmsnorm (bf16 out)", "reference", M, timeit(lambda i: ref_rms_norm(x, w_ln, o)), M * H * 4)
        report("rmsnorm (bf16 out)", "in-tree", M, timeit(lambda i: ops.row_op(x, "bf16", ops.IN_RMSNORM, w=w_ln, plus_one=True)), M * H * 4)
        report("rmsnorm (bf16 out)", "torch", M, timeit(lambda i: torch.nn.functional.rms_norm(x, (H,), w_ln + 1, 1e-6)), M * H * 4)
        report("rmsnorm + nvfp4 quant", "in-tree", M, timeit(lambda i: ops.row_op(x, "nvfp4", ops.IN_RMSNORM, w=w_ln, plus_one=True)), M * H * 2.6)
        # the four per-layer GEMMs: reference W4A16 (bf16 activations), in-tree W4A4 tcgen05, torch bf16 (cuBLAS)
        for name, N, K in (("qkv", (Hq + 2 * Hkv) * D, H), ("o_proj", H, Hq * D), ("gate_up", 2 * I, H), ("down", H, I)):
            copies = max(2, int(400e6 // (N * K * 0.5625)) + 1)
            packed = [torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=DEV) for _ in range(copies)]
            scale = [torch.randint(40, 60, (N, K // 16), dtype=torch.uint8, device=DEV) for _ in range(copies)]
            a16 = torch.randn(M, K, device=DEV).to(torch.bfloat16)
            oo = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
            wb = N * K * 0.5625 + M * K * 2 + M * N * 2
            report(f"gemm {name}", "reference", M, timeit(lambda i: ref_w4a16(a16, packed[i % copies], scale[i % copies], 1e-3, oo)), wb)
            ws = []
            for c in range(copies):
                qw = ops.QuantWeight("nvfp4", N, K, packed[c], scale[c], 1e-3)
                qw.prepare_cuda()
                ws.append(qw)
            act = ops.quantize_act(a16, "nvfp4")
            report(f"gemm {name}", "in-tree", M, timeit(lambda i: ops.linear(act, ws[i % copies], out=oo)), wb)
            del ws, packed, scale
            cb = max(2, int(400e6 // (N * K * 2)) + 1)
            wbf = [(torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(cb)]
            report(f"gemm {name}", "torch-bf16", M, timeit(lambda i: torch.matmul(a16, wbf[i % cb].t(), out=oo)),
                   N * K * 2 + M * K * 2 + M * N * 2)
            del wbf
        # lm_head (bf16) + argmax
        if M <= 16:
            wl = [(torch.randn(V, H, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(2)]
            lo = torch.empty(M, V, device=DEV, dtype=torch.bfloat16)
            lb = V * H * 2 + M * V * 2
            report("lm_head", "reference", M, timeit(lambda i: ref_dense_gemv(x, wl[i % 2], lo), iters=6), lb)
            qwl = [ops.QuantWeight("bf16", V, H, t) for t in wl]
            act = ops.quantize_act(x, "bf16")
            report("lm_head", "in-tree", M, timeit(lambda i: ops.linear(act, qwl[i % 2], out=lo), iters=6), lb)
            report("lm_head", "torch-bf16", M, timeit(lambda i: torch.matmul(x, wl[i % 2].t(), out=lo), iters=6), lb)
            ids = torch.zeros(M, dtype=torch.int32, device=DEV)
            report("argmax", "reference", M, timeit(lambda i: ref_argmax(lo, ids)), M * V * 2)
            report("argmax", "in-tree", M, timeit(lambda i: ops.argmax(lo, out=ids)), M * V * 2)
            report("argmax", "torch", M, timeit(lambda i: torch.argmax(lo, dim=-1)), M * V * 2)
            del wl, qwl
        # decode attention, fp8 KV, M sequences at ctx tokens
        ctx, bs = args.ctx, 16
        nblk = (ctx + bs - 1) // bs
        kc = torch.randint(0x20, 0x48, (M * nblk + 1, bs, Hkv, D), dtype=torch.uint8, device=DEV)
        vc = torch.randint(0x20, 0x48, (M * nblk + 1, bs, Hkv, D), dtype=torch.uint8, device=DEV)
        bt = torch.zeros(M, 128, dtype=torch.int32, device=DEV)
        bt[:, :nblk] = (torch.arange(M * nblk, device=DEV, dtype=torch.int32) + 1).view(M, nblk)
        q = torch.randn(M, Hq, D, device=DEV).to(torch.bfloat16)
        sl = torch.full((M,), ctx, dtype=torch.int32, device=DEV)
        ao = torch.empty_like(q)
        ab = 2.0 * M * ctx * Hkv * D
        report(f"decode attn fp8 ctx={ctx}", "reference", M, timeit(lambda i: ref_decode_attn(q, kc, vc, ao, bt, sl, 0.05, 0.05)), ab)
        qs = torch.arange(M, device=DEV, dtype=torch.int32)
        ql = torch.ones(M, device=DEV, dtype=torch.int32)
        sc = torch.tensor([0.05], device=DEV)
        report(f"decode attn fp8 ctx={ctx}", "in-tree", M,
               timeit(lambda i: ops.paged_attention(q, kc, vc, bt, qs, ql, sl, max_q_len=1, max_ctx=2048,
                                                    scale=1 / math.sqrt(D), k_scale=sc, v_scale=sc)), ab)
        kd = torch.randn(M, Hkv, ctx, D, device=DEV).to(torch.bfloat16)
        vd = torch.randn(M, Hkv, ctx, D, device=DEV).to(torch.bfloat16)
        qd = q.view(M, Hq, 1, D)
        report(f"decode attn bf16 ctx={ctx}", "torch-sdpa", M,
               timeit(lambda i: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, enable_gqa=True)),
               2.0 * M * ctx * Hkv * D * 2)
    if args.json:
        json.dump({"peaks": {"hbm_gbs": hbm, "tag": tag}, "rows": rows}, open(args.json, "w"), indent=1)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--build", action="store_true")
    ap.add_argument("--run", action="store_true")
    ap.add_argument("--reference-root", default=os.environ.get("METRALE_REFERENCE_ROOT", "/root/reference"))
    ap.add_argument("--m", default="1,16,128")
    ap.add_argument("--ctx", type=int, default=640)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    rc = 0
    if args.build:
        rc = build(args.reference_root)
    if args.run:
        rc = rc or run(args)
    if not (args.build or args.run):
        ap.print_help()
    return rc


if __name__ == "__main__":
    sys.exit(main())
