"""Vision tower of the Qwen-VL family: patch embedding, ViT blocks with 2-D rotary positions and
attention confined to each frame, and the 2x2 patch merger that emits one LLM-width embedding per
merged patch.

Input is the flattened patch matrix the preprocessor produces (``[N, C * Tp * P * P]``, patches ordered
so that each merge group is contiguous) plus ``grid_thw`` (frames, patch rows, patch columns per image).
Weights use the HF tensor names of ``Qwen2VisionTransformerPretrainedModel`` (``visual.`` prefix
stripped): ``patch_embed.proj.weight``, ``blocks.N.{norm1,norm2,attn.qkv,attn.proj,mlp.fc1,mlp.fc2}``,
``merger.{ln_q,mlp.0,mlp.2}``.

The GEMMs go through ``ops.linear`` (the tcgen05 bf16 kernel on a GPU); LayerNorm, the rotary rotation,
the activation and the per-frame attention are PyTorch ops: the tower runs once per image at prefill
and is a small fraction of a request. Reference: ``kernels/gb10/qwen3-vl-30b-a3b/nvfp4/vision_encoder.cu``
(patch embed / attention / merger kernels) and the vision stack of ``crates/model-layers``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


@dataclass
class VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584            # LLM width (merger output)
    num_heads: int = 16
    mlp_ratio: float = 4.0
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    hidden_act: str = "quick_gelu"
    eps: float = 1e-6

    @staticmethod
    def from_hf(d: dict) -> "VisionConfig":
        keys = VisionConfig.__dataclass_fields__
        return VisionConfig(**{k: d[k] for k in keys if k in d})

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2


def _act(x: torch.Tensor, kind: str) -> torch.Tensor:
    if kind == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if kind in ("gelu", "gelu_pytorch_tanh"):
        return F.gelu(x, approximate="tanh" if kind == "gelu_pytorch_tanh" else "none")
    if kind == "silu":
        return F.silu(x)
    raise ValueError(f"unsupported vision activation {kind!r}")


def rot_pos_ids(grid_thw: torch.Tensor, merge: int) -> torch.Tensor:
    """(row, column) of every patch in preprocessor order: inside an image the patches of one merge group
    are contiguous, groups run row-major, frames repeat the same grid. [N, 2] int64."""
    out = []
    for t, h, w in grid_thw.tolist():
        hp = torch.arange(h)[:, None].expand(h, w).reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten()
        wp = torch.arange(w)[None, :].expand(h, w).reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten()
        out.append(torch.stack([hp, wp], -1).repeat(t, 1))
    return torch.cat(out, 0)


def rotary_cos_sin(grid_thw: torch.Tensor, head_dim: int, merge: int, theta: float = 10000.0, device="cpu"):
    """cos / sin [N, head_dim] of the 2-D rotary embedding: a quarter of the head rotates with the patch
    row, a quarter with its column, and the table is repeated for the two halves of rotate_half."""
    dim = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    pos = rot_pos_ids(grid_thw, merge)
    freqs = torch.outer(torch.arange(int(grid_thw[:, 1:].max()), dtype=torch.float32), inv)       # [grid, dim / 2]
    emb = freqs[pos].flatten(1)                                                                    # [N, dim]
    emb = torch.cat([emb, emb], -1)
    return emb.cos().to(device), emb.sin().to(device)


def _rotate_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([-b, a], -1)


class VisionEncoder:
    def __init__(self, cfg: VisionConfig, tensors: Dict[str, torch.Tensor], device="cpu"):
        from ..ops import QuantWeight
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        t = {k: v.to(self.device) for k, v in tensors.items()}

        def lin(name):
            w = t[name + ".weight"]
            w = w.reshape(w.shape[0], -1)
            qw = QuantWeight("bf16", w.shape[0], w.shape[1], w.to(torch.bfloat16).contiguous()) if self.device.type == "cuda" else w.float()
            b = t.get(name + ".bias")
            return qw, (None if b is None else b.float())

        self.patch = lin("patch_embed.proj")
        self.blocks = []
        for i in range(cfg.depth):
            p = f"blocks.{i}"
            self.blocks.append(dict(n1=(t[f"{p}.norm1.weight"].float(), t[f"{p}.norm1.bias"].float()),
                                    n2=(t[f"{p}.norm2.weight"].float(), t[f"{p}.norm2.bias"].float()),
                                    qkv=lin(f"{p}.attn.qkv"), proj=lin(f"{p}.attn.proj"),
                                    fc1=lin(f"{p}.mlp.fc1"), fc2=lin(f"{p}.mlp.fc2")))
        self.ln_q = (t["merger.ln_q.weight"].float(), t["merger.ln_q.bias"].float())
        self.m0, self.m2 = lin("merger.mlp.0"), lin("merger.mlp.2")

    @staticmethod
    def random_tensors(cfg: VisionConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: torch.randn(*s, generator=g) * 0.05
        E, M = cfg.embed_dim, int(cfg.embed_dim * cfg.mlp_ratio)
        t = {"patch_embed.proj.weight": r(E, cfg.in_channels, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size)}
        for i in range(cfg.depth):
            p = f"blocks.{i}"
            for n in ("norm1", "norm2"):
                t[f"{p}.{n}.weight"], t[f"{p}.{n}.bias"] = 1 + r(E), r(E)
            for n, (o, k) in {"attn.qkv": (3 * E, E), "attn.proj": (E, E), "mlp.fc1": (M, E), "mlp.fc2": (E, M)}.items():
                t[f"{p}.{n}.weight"], t[f"{p}.{n}.bias"] = r(o, k), r(o)
        m2 = cfg.spatial_merge_size ** 2
        t["merger.ln_q.weight"], t["merger.ln_q.bias"] = 1 + r(E), r(E)
        t["merger.mlp.0.weight"], t["merger.mlp.0.bias"] = r(E * m2, E * m2), r(E * m2)
        t["merger.mlp.2.weight"], t["merger.mlp.2.bias"] = r(cfg.hidden_size, E * m2), r(cfg.hidden_size)
        return t

    def _linear(self, x: torch.Tensor, wb) -> torch.Tensor:
        w, b = wb
        if self.device.type == "cuda":
            from .. import ops
            xa = x.to(torch.bfloat16).contiguous()
            y = ops.linear(ops.Act("bf16", xa.shape[0], xa.shape[1], xa, bf16=xa), w, out_f32=True)
        else:
            y = x.float() @ w.T
        return y if b is None else y + b

    def __call__(self, patches: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """``patches`` [N, patch_dim] -> merged embeddings [N / merge^2, hidden_size] (fp32)."""
        c = self.cfg
        if patches.shape[1] != c.patch_dim:
            raise ValueError(f"patch rows have {patches.shape[1]} values, the tower expects {c.patch_dim}")
        n_exp = int((grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).sum())
        if patches.shape[0] != n_exp:
            raise ValueError(f"{patches.shape[0]} patches for grids that hold {n_exp}")
        x = self._linear(patches.to(self.device), self.patch)                       # [N, E]
        cos, sin = rotary_cos_sin(grid_thw, c.head_dim, c.spatial_merge_size, device=self.device)
        # attention never crosses a frame: one segment per (image, frame)
        seg = torch.repeat_interleave(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0]).tolist()
        H, D = c.num_heads, c.head_dim
        for blk in self.blocks:
            h = F.layer_norm(x, (c.embed_dim,), *blk["n1"], c.eps)
            qkv = self._linear(h, blk["qkv"]).view(-1, 3, H, D)
            q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
            q = q * cos[:, None] + _rotate_half(q) * sin[:, None]
            k = k * cos[:, None] + _rotate_half(k) * sin[:, None]
            outs, s0 = [], 0
            for n in seg:
                qs, ks, vs = (z[s0:s0 + n].transpose(0, 1) for z in (q, k, v))          # [H, n, D]
                outs.append(F.scaled_dot_product_attention(qs[None], ks[None], vs[None])[0].transpose(0, 1))
                s0 += n
            a = torch.cat(outs, 0).reshape(-1, c.embed_dim)
            x = x + self._linear(a, blk["proj"])
            h = F.layer_norm(x, (c.embed_dim,), *blk["n2"], c.eps)
            x = x + self._linear(_act(self._linear(h, blk["fc1"]), c.hidden_act), blk["fc2"])
        m2 = c.spatial_merge_size ** 2
        h = F.layer_norm(x, (c.embed_dim,), *self.ln_q, c.eps).view(-1, c.embed_dim * m2)
        return self._linear(F.gelu(self._linear(h, self.m0)), self.m2)
