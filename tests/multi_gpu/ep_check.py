"""2+ ranks: expert-parallel MoE through the peer-memory all-to-all (parallel/ep.py) against the
masked-local + all-reduce scheme on the same synthetic checkpoint, at decode- and prefill-sized
batches, for several consecutive steps (both parities). Launched by tests/test_tp_gpu.py."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from metrale_inference_alpha_b200 import ops  # noqa: E402
from metrale_inference_alpha_b200.config.model_config import preset  # noqa: E402
from metrale_inference_alpha_b200.models.decoder import Decoder  # noqa: E402
from metrale_inference_alpha_b200.models.moe import moe_block  # noqa: E402
from metrale_inference_alpha_b200.parallel.ep import EpAllToAll  # noqa: E402
from metrale_inference_alpha_b200.parallel.tp import NcclTpContext  # noqa: E402
from metrale_inference_alpha_b200.weights.loader import load_weights  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    cfg = preset("qwen-hybrid-moe-35b-fp8", num_layers=1, hidden_size=512, num_heads=4, num_kv_heads=2,
                 gdn_k_heads=4, gdn_v_heads=4, num_experts=8, experts_per_token=2, moe_intermediate_size=256,
                 intermediate_size=256, vocab_size=4096, max_position=256, layer_types=["attention"], ffn_types=["moe"])
    tp = NcclTpContext(rank, world, dev, fused=False)
    tp.ep_rank = rank
    w = load_weights(cfg, None, device=dev, tp_rank=0, tp_size=1, ep_rank=rank, ep_size=world, seed=0)
    dec = Decoder(cfg, w, tp, dev)
    lw = w.layers[0]
    ep = EpAllToAll(rank, world, dev, hidden=cfg.hidden_size, max_tokens=128, top_k=cfg.experts_per_token)
    ok = True
    for step, T in enumerate((1, 7, 64, 128, 3)):
        g = torch.Generator(device="cpu").manual_seed(100 + step)
        x = (torch.randn(T, cfg.hidden_size, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        tp.ep = None
        want = moe_block(dec, x, lw)
        tp.ep = ep
        got = moe_block(dec, x, lw)
        torch.cuda.synchronize()
        ops.check_status(dev)
        err = (got.float() - want.float()).abs().max().item()
        ref = want.float().abs().max().item()
        good = err <= 3e-2 * max(1.0, ref)
        ok = ok and good
        if rank == 0:
            print(f"T={T:4d} max err {err:.4g} (ref {ref:.3g}) {'ok' if good else 'MISMATCH'}", flush=True)
    # the same exchange inside a CUDA graph, replayed: the sequence number comes from device memory,
    # so every replay publishes and waits for a fresh value
    tp.ep = ep
    xs = (torch.randn(16, cfg.hidden_size, generator=torch.Generator().manual_seed(9)) * 0.5).to(torch.bfloat16).to(dev)
    for _ in range(2):
        moe_block(dec, xs, lw)                                    # warm-up outside the capture
    torch.cuda.synchronize()
    dist.barrier()
    gph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gph):
        y1 = moe_block(dec, xs, lw)
        y2 = moe_block(dec, y1.to(torch.bfloat16), lw)               # two exchanges per replay (both parities)
    tp.ep = None
    want1 = moe_block(dec, xs, lw)
    want2 = moe_block(dec, want1.to(torch.bfloat16), lw)
    for rep in range(3):
        gph.replay()
        torch.cuda.synchronize()
        ops.check_status(dev)
        err = (y2.float() - want2.float()).abs().max().item()
        ref = want2.float().abs().max().item()
        good = err <= 3e-2 * max(1.0, ref)
        ok = ok and good
        if rank == 0:
            print(f"graph replay {rep}: max err {err:.4g} (ref {ref:.3g}) {'ok' if good else 'MISMATCH'}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_CHECK PASS" if int(flag) else "EP_CHECK FAIL", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
