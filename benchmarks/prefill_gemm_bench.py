#!/usr/bin/env python
"""Times the four projection GEMMs of the dense 27B layer at a prefill-sized token count (several
128-token tiles), NVFP4 and bf16, with CUDA events over 10 launches after 3 warm-up launches.

    python benchmarks/prefill_gemm_bench.py --m 8192
    METRALE_PERSISTENT_PREFILL=0 python benchmarks/prefill_gemm_bench.py --m 8192    # one tile per CTA
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from metrale_inference_alpha_b200 import ops  # noqa: E402
from kernel_bench import rand_weight  # noqa: E402

DEV = "cuda"
SHAPES = [("qkv", 7168, 5120, False), ("o_proj", 5120, 5120, False), ("gate_up+swiglu", 34816, 5120, True),
          ("down", 5120, 17408, False)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--fmt", default="nvfp4,bf16")
    a = ap.parse_args()
    torch.manual_seed(0)
    for fmt in a.fmt.split(","):
        for name, N, K, swiglu in SHAPES:
            w = rand_weight(N, K, fmt, 1)[0]
            if swiglu:                                        # rows interleaved (gate_j, up_j) as the loader stores them
                perm = torch.stack([torch.arange(N // 2), torch.arange(N // 2) + N // 2], 1).reshape(-1).to(DEV)
                w = ops.permute_rows(w, perm)
                if fmt == "nvfp4":
                    w.prepare_cuda()
            x = torch.randn(a.m, K, device=DEV).to(torch.bfloat16)
            act = ops.quantize_act(x, ops.ACT_FOR_WEIGHT[fmt])
            for _ in range(3):
                ops.linear(act, w, swiglu=swiglu)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                ops.linear(act, w, swiglu=swiglu)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            print(f"{fmt:6s} {name:16s} M={a.m:6d}  {ms * 1e3:9.1f} us  {2 * a.m * N * K / ms / 1e9:7.0f} TFLOP/s", flush=True)
    ops.check_status(DEV)


if __name__ == "__main__":
    main()
