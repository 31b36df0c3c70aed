"""Run under torchrun on >= 2 GPUs: checks the fused GEMM + all-reduce kernel against the NCCL
baseline (local GEMM, then ncclAllReduce), eagerly and inside a CUDA graph, and times both with
CUDA events (max over ranks).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        tests/multi_gpu/tp_check.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from metrale_inference_alpha_b200 import ops  # noqa: E402
from metrale_inference_alpha_b200.parallel.tp import NcclTpContext  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    os.environ["METRALE_NVLS"] = "2"                        # reduction inside the switch (multimem.ld_reduce)
    tp = NcclTpContext(rank, world, dev, fused=True)
    os.environ.pop("METRALE_NVLS")
    assert tp.fused, "fused collectives did not initialise"
    base = NcclTpContext(rank, world, dev, fused=False)
    # the same fused kernel with one peer store per rank instead of NVLink multicast stores
    os.environ["METRALE_NVLS"] = "0"
    p2p = NcclTpContext(rank, world, dev, fused=True)
    os.environ["METRALE_NVLS"] = "1"
    mcst = NcclTpContext(rank, world, dev, fused=True)      # multicast stores, reduction on every rank
    os.environ.pop("METRALE_NVLS")
    assert p2p.fused and not p2p.fused_impl.nvls and mcst.fused and not mcst.fused_impl.in_switch
    if rank == 0:
        print(f"fused path: nvls multicast {'on' if tp.fused_impl.nvls else 'unavailable (peer stores)'}, "
              f"in-switch reduction {'on' if tp.fused_impl.in_switch else 'off'}", flush=True)
    ok = True
    for fmt in ("nvfp4", "bf16"):
        for (M, N, Kfull) in ((1, 5120, 5120), (16, 5120, 17408), (128, 5120, 17408), (100, 2048, 4096)):
            K = Kfull // world
            K -= K % 256
            g = torch.Generator().manual_seed(100 + rank)
            w = ops.make_weight(torch.randn(N, K, generator=g) * 0.05, fmt).to(dev)
            x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
            res = torch.randn(M, N, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(dev)
            act = ops.quantize_act(x, ops.ACT_FOR_WEIGHT[fmt])
            want = base.linear_reduce(act, w, residual=res).float()
            for name, ctx in (("in-switch" if tp.fused_impl.in_switch else "p2p", tp), ("mc-stores", mcst), ("p2p", p2p)):
                for it in range(3):
                    got = ctx.linear_reduce(act, w, residual=res).float().clone()
                    torch.cuda.synchronize()
                    err = (got - want).abs().max().item()
                    tol = 0.03 * max(1.0, want.abs().max().item())
                    if err > tol:
                        ok = False
                        print(f"[r{rank}] MISMATCH {name} {fmt} M={M} N={N} K={K} it={it} err={err:.4f} tol={tol:.4f}", flush=True)
            ops.check_status(dev)
            # timing inside CUDA graphs
            def timed(ctx):
                for _ in range(3):
                    ctx.linear_reduce(act, w, residual=res)
                torch.cuda.synchronize()
                dist.barrier()
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph):
                    for _ in range(10):
                        ctx.linear_reduce(act, w, residual=res)
                gph.replay()
                torch.cuda.synchronize()
                dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(5):
                    gph.replay()
                b.record()
                torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b) / 50 * 1e3], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return t.item()
            t_fused = timed(tp)
            t_p2p = timed(p2p)
            t_mc = timed(mcst)
            t_nccl = timed(base)
            ops.check_status(dev)
            if rank == 0:
                print(f"{fmt} M={M} N={N} K/rank={K}: fused {t_fused:.2f} us  fused(multicast stores) {t_mc:.2f} us  fused(peer stores) {t_p2p:.2f} us  "
                      f"gemm+nccl {t_nccl:.2f} us  speedup {t_nccl / t_fused:.2f}x", flush=True)
    dist.barrier()
    if rank == 0:
        print("TP_CHECK", "PASS" if ok else "FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
