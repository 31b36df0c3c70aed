"""Run under torchrun on >= 2 GPUs: checks the consumer-fused tensor-parallel reduction
(row-parallel GEMM -> [all-reduce + residual + RMSNorm + NVFP4 quantiser (+ all-gather)] in one
kernel) against the NCCL baseline (GEMM, ncclAllReduce, separate norm + quantiser kernel),
eagerly and inside a CUDA graph, times both with CUDA events (max over ranks), and checks the
vocabulary-parallel argmax merge against an all-gather of the logits.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        tests/multi_gpu/tp_check.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from metrale_inference_alpha_b200 import ops  # noqa: E402
from metrale_inference_alpha_b200.ops import reference as ref  # noqa: E402
from metrale_inference_alpha_b200.parallel.tp import NcclTpContext  # noqa: E402


def deq_nvfp4(a, M, K):
    nb = (M + 127) // 128
    sf = ref.tiled_to_sf(a.sf.cpu()[:nb * a.sf_k64 * 512].view(nb, a.sf_k64, 512), M, K // 16)
    return ref.dequantize_nvfp4(a.data.cpu(), sf, a.scale.cpu())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    N = 5120
    tp = NcclTpContext(rank, world, dev, fused=True)
    assert tp.setup_fused(N, 512), "fused reduction did not initialise"
    base = NcclTpContext(rank, world, dev, fused=False)
    fr = tp.reduce
    if rank == 0:
        print(f"fused reduction: multicast {'on' if fr.mc else 'off (peer loads, one-shot only)'}, "
              f"one-shot up to {fr.one_shot_bytes} bytes served per GPU", flush=True)
    ok = True
    gw = torch.Generator().manual_seed(3)
    wn = (torch.randn(N, generator=gw) * 0.1).to(torch.bfloat16).to(dev)
    for fmt in ("nvfp4",):
        for (M, Kfull) in ((1, 5120), (8, 17408), (16, 17408), (32, 17408), (64, 17408), (128, 17408), (300, 5120)):
            K = Kfull // world
            K -= K % 256
            g = torch.Generator().manual_seed(100 + rank)
            w = ops.make_weight(torch.randn(N, K, generator=g) * 0.05, fmt).to(dev)
            x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
            res = torch.randn(M, N, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(dev)
            act = ops.quantize_act(x, ops.ACT_FOR_WEIGHT[fmt])

            def baseline():
                y = base.linear_reduce(act, w, residual=res)
                return ops.row_op(y, "nvfp4", ops.IN_RMSNORM, w=wn, eps=1e-6, also_bf16=True)[0], y

            def fused(res_only=False):
                p = tp.linear_reduce(act, w, residual=res, defer=True)
                a = fr.reduce_norm(p, wn, "nvfp4", eps=1e-6, also_bf16=True, gather_residual=not res_only)
                return a, p.value

            a0, y0 = baseline()
            want_bf16, want_res, want_deq = a0.bf16.float().cpu(), y0.float().cpu(), deq_nvfp4(a0, M, N)
            protos = [0] + ([1] if fr.mc else []) + ([2] if M <= fr.ll_rows else [])
            for it in range(3 * len(protos)):
                fr.force_proto = protos[it % len(protos)]
                a1, y1 = fused()
                fr.force_proto = None
                torch.cuda.synchronize()
                e_res = (y1.float().cpu() - want_res).abs().max().item()
                e_n = (a1.bf16.float().cpu() - want_bf16).abs().max().item()
                dq = deq_nvfp4(a1, M, N)
                # one e2m1 step at the top of the range is a third of the row maximum
                step = want_deq.abs().amax(dim=1, keepdim=True) * 0.35
                frac = ((dq - want_deq).abs() > 1e-3).float().mean().item()
                bad = not ((dq - want_deq).abs() <= step + 1e-3).all().item()
                # the residual stream may differ by bf16 roundings of the cross-rank sum (NCCL and the
                # switch add the ranks' bf16 partials in different orders): two ulps of the largest value
                if e_res > 2 ** -6 * max(1.0, want_res.abs().max().item()) or e_n > 0.08 or bad or frac > 0.2:
                    ok = False
                    print(f"[r{rank}] MISMATCH proto={protos[it % len(protos)]} M={M} K={K} it={it} e_res={e_res:.4f} e_norm={e_n:.4f} "
                          f"quant_bad={bad} frac={frac:.3f}", flush=True)
            tp.end_forward()
            ops.check_status(dev)

            def timed(fn):
                for _ in range(3):
                    fn()
                tp.end_forward()
                torch.cuda.synchronize()
                dist.barrier()
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph):
                    for _ in range(10):
                        fn()
                    tp.end_forward()
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
            fr.force_proto = 0
            t_one = timed(lambda: fused(True))
            fr.force_proto = 1
            t_two = timed(lambda: fused(True)) if fr.mc else float("nan")
            fr.force_proto = 2
            t_pkt = timed(lambda: fused(True)) if M <= fr.ll_rows else float("nan")
            fr.force_proto = None
            t_fused = timed(lambda: fused(True))
            t_nccl = timed(baseline)
            t_gemm = timed(lambda: ops.linear(act, w, residual=res))
            ops.check_status(dev)
            if rank == 0:
                print(f"{fmt} M={M} N={N} K/rank={K}: gemm+fused(reduce,residual,norm,quant,gather) {t_fused:.2f} us (protocol {fr.protocol(M, N)}: one-shot {t_one:.2f}, two-shot {t_two:.2f}, packets {t_pkt:.2f})   "
                      f"gemm+nccl+norm-quant {t_nccl:.2f} us   gemm alone {t_gemm:.2f} us   speedup {t_nccl / t_fused:.2f}x",
                      flush=True)
    # vocabulary-parallel greedy selection
    V = 18992
    for M in (1, 128):
        g = torch.Generator().manual_seed(55 + rank)
        lg = torch.randn(M, V, generator=g).to(torch.bfloat16).to(dev)
        out = torch.zeros(M, dtype=torch.int32, device=dev)
        fr.argmax_merge(lg, rank * V, out)
        want = ops.argmax(base.all_gather_last(lg))
        torch.cuda.synchronize()
        if not torch.equal(out, want):
            ok = False
            print(f"[r{rank}] argmax merge mismatch M={M}", flush=True)
    ops.check_status(dev)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_CHECK", "PASS" if flag.item() else "FAIL", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
