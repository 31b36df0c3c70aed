"""Library baseline for the headline benchmark (`bench.py --impl torch`): the same dense
decoder shape, batch and context, built from PyTorch's stock kernels only: cuBLAS bf16 GEMMs
(`torch.matmul`), `F.rms_norm`, `F.scaled_dot_product_attention` over a contiguous bf16 KV
cache, and NCCL all-reduces after the row-parallel projections for tensor parallelism (the
reference's collective placement). Weights are random bf16 of the named architecture (the NVFP4
checkpoint dequantised would have the same shapes; library GEMMs have no NVFP4 x NVFP4 path
here). One decode step at a fixed context is captured in a CUDA graph and replayed K times
between CUDA events, which is the same measurement as the `value` of the in-tree arm.

None of the in-tree kernels, models or engine code is on this path.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F


class TorchDecoder:
    def __init__(self, cfg, batch: int, max_ctx: int, rank: int, world: int, device: str, seed: int = 0):
        self.cfg, self.B, self.rank, self.world, self.dev = cfg, batch, rank, world, device
        H, D = cfg.hidden_size, cfg.head_dim
        self.hq, self.hkv = cfg.num_heads // world, max(1, cfg.num_kv_heads // world)
        inter = cfg.intermediate_size // world
        g = torch.Generator(device=device).manual_seed(seed + rank)

        def w(n, k):
            return (torch.randn(n, k, device=device, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append(dict(
                ln1=torch.ones(H, device=device, dtype=torch.bfloat16), ln2=torch.ones(H, device=device, dtype=torch.bfloat16),
                qkv=w((self.hq + 2 * self.hkv) * D, H), o=w(H, self.hq * D), gate_up=w(2 * inter, H), down=w(H, inter),
                qn=torch.ones(D, device=device, dtype=torch.bfloat16), kn=torch.ones(D, device=device, dtype=torch.bfloat16),
                k=torch.zeros(batch, self.hkv, max_ctx, D, device=device, dtype=torch.bfloat16),
                v=torch.zeros(batch, self.hkv, max_ctx, D, device=device, dtype=torch.bfloat16)))
        self.embed = w(cfg.vocab_size, H)
        vs = (cfg.vocab_size + world - 1) // world
        self.lm_head = w(vs, H)
        self.final = torch.ones(H, device=device, dtype=torch.bfloat16)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, device=device).float() / D))
        t = torch.arange(max_ctx, device=device).float()
        fr = torch.outer(t, inv)
        self.cos, self.sin = fr.cos().to(torch.bfloat16), fr.sin().to(torch.bfloat16)
        self.inter = inter

    def weight_bytes(self) -> int:
        n = self.embed.numel() + self.lm_head.numel()
        for l in self.layers:
            n += l["qkv"].numel() + l["o"].numel() + l["gate_up"].numel() + l["down"].numel()
        return n * 2

    def _rope(self, x, pos):
        # x [B, heads, D], NeoX halves
        D = x.shape[-1]
        c, s = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        x1, x2 = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    def step(self, tokens: torch.Tensor, pos: torch.Tensor, ctx: int) -> torch.Tensor:
        """One decode step for the whole batch: tokens [B], pos [B] (all equal to ctx - 1)."""
        cfg, D, B = self.cfg, self.cfg.head_dim, self.B
        x = self.embed[tokens]
        bi = torch.arange(B, device=self.dev)
        for l in self.layers:
            h = F.rms_norm(x, (cfg.hidden_size,), l["ln1"], cfg.rms_eps)
            qkv = h @ l["qkv"].t()
            q = qkv[:, :self.hq * D].view(B, self.hq, D)
            k = qkv[:, self.hq * D:(self.hq + self.hkv) * D].view(B, self.hkv, D)
            v = qkv[:, (self.hq + self.hkv) * D:].view(B, self.hkv, D)
            q = self._rope(F.rms_norm(q, (D,), l["qn"], cfg.rms_eps), pos)
            k = self._rope(F.rms_norm(k, (D,), l["kn"], cfg.rms_eps), pos)
            l["k"][bi, :, pos] = k
            l["v"][bi, :, pos] = v
            o = F.scaled_dot_product_attention(q.unsqueeze(2), l["k"][:, :, :ctx], l["v"][:, :, :ctx], enable_gqa=True)
            y = o.reshape(B, self.hq * D) @ l["o"].t()
            if self.world > 1:
                dist.all_reduce(y)
            x = x + y
            h = F.rms_norm(x, (cfg.hidden_size,), l["ln2"], cfg.rms_eps)
            gu = h @ l["gate_up"].t()
            a = F.silu(gu[:, :self.inter]) * gu[:, self.inter:]
            y = a @ l["down"].t()
            if self.world > 1:
                dist.all_reduce(y)
            x = x + y
        h = F.rms_norm(x, (cfg.hidden_size,), self.final, cfg.rms_eps)
        lg = h @ self.lm_head.t()
        if self.world > 1:
            parts = [torch.empty_like(lg) for _ in range(self.world)]
            dist.all_gather(parts, lg)
            lg = torch.cat(parts, -1)
        return lg.argmax(-1)


def run(cfg, concurrency: int, ctx: int, steps: int, warmup: int, rank: int, world: int, device: str) -> dict:
    """K graph-replayed decode steps at `ctx`; returns tok/s (whole job), ms/step and launches."""
    model = TorchDecoder(cfg, concurrency, ctx + 8, rank, world, device)
    tokens = torch.randint(0, cfg.vocab_size, (concurrency,), device=device)
    pos = torch.full((concurrency,), ctx - 1, device=device, dtype=torch.long)
    for l in model.layers:                             # a filled cache: random keys / values up to ctx
        l["k"].normal_()
        l["v"].normal_()
    for _ in range(2):
        model.step(tokens, pos, ctx)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = model.step(tokens, pos, ctx)
    for _ in range(max(3, warmup)):
        g.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    sec = a.elapsed_time(b) / 1e3
    if world > 1:
        t = torch.tensor([sec], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return dict(tok_s=concurrency * steps / sec, ms_per_step=sec / steps * 1e3, weight_bytes=model.weight_bytes(),
                sample=int(out[0].item()))
