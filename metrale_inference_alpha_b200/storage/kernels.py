"""Device ops of the KV storage tier (``ops/csrc/storage.cu``) and their fp32 restatements.

Every function takes CUDA tensors and launches the kernel, or takes CPU tensors and runs the plain
PyTorch form (the oracle of the GPU tests and the path of the CPU tests). Pools are addressed by
element strides ``(blk, tok, kvh)`` so that one kernel reads the engine's paged cache
``[blocks, block, kv_heads, D]`` and the scratch pool's ``[slot, K|V, block, kv_heads, D]`` alike.

Reference: ``crates/storage/kernels/*.cu`` and their host sides ``crates/storage/src/predictor.rs``,
``tiled_attention.rs``; oracles ``attention_ref.rs`` / ``predictor_ref.rs``.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from ..ops import _native

c_void_p, c_int, c_ll, c_float = C.c_void_p, C.c_int, C.c_longlong, C.c_float


class KvTileArgs(C.Structure):
    _fields_ = [("q", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("tile_blocks", c_void_p),
                ("tile_counts", c_void_p), ("last_valid", c_void_p), ("m_state", c_void_p), ("l_state", c_void_p),
                ("o_state", c_void_p), ("out", c_void_p),
                ("num_seqs", c_int), ("Hq", c_int), ("Hkv", c_int), ("D", c_int), ("block_size", c_int),
                ("cap", c_int), ("kv_fp8", c_int),
                ("blk_stride", c_ll), ("tok_stride", c_ll), ("kvh_stride", c_ll),
                ("scale", c_float), ("k_scale", c_float), ("v_scale", c_float)]


class LowrankArgs(C.Structure):
    _fields_ = [("x", c_void_p), ("P", c_void_p), ("out", c_void_p), ("src_blocks", c_void_p),
                ("dst_blocks", c_void_p), ("rows", c_ll),
                ("D", c_int), ("r", c_int), ("Hkv", c_int), ("block_size", c_int), ("fp8", c_int),
                ("blk_stride", c_ll), ("tok_stride", c_ll), ("kvh_stride", c_ll), ("scale", c_float)]


class ScoreArgs(C.Structure):
    _fields_ = [("q_lr", c_void_p), ("k_lr", c_void_p), ("blocks", c_void_p), ("counts", c_void_p),
                ("last_valid", c_void_p), ("scores", c_void_p),
                ("num_seqs", c_int), ("Hq", c_int), ("Hkv", c_int), ("block_size", c_int), ("r", c_int),
                ("cap", c_int)]


_native.register_optional("mb_kv_tile_attn", [C.POINTER(KvTileArgs), c_void_p])
_native.register_optional("mb_attn_finalize", [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p])
_native.register_optional("mb_lowrank_project", [C.POINTER(LowrankArgs), c_void_p])
_native.register_optional("mb_predictor_score", [C.POINTER(ScoreArgs), c_void_p])

Strides = Tuple[int, int, int]


def paged_strides(block_size: int, kv_heads: int, head_dim: int) -> Strides:
    """Element strides of a pool laid out ``[blocks, block, kv_heads, D]``."""
    return block_size * kv_heads * head_dim, kv_heads * head_dim, head_dim


def _is_fp8(t: torch.Tensor) -> bool:
    return t.dtype in (torch.float8_e4m3fn, torch.uint8)


def _widen(t: torch.Tensor, scale: float) -> torch.Tensor:
    if t.dtype == torch.uint8:
        t = t.view(torch.float8_e4m3fn)
    f = t.float()
    return f * scale if _is_fp8(t) else f


def _rows(pool: torch.Tensor, strides: Strides, blk: int, kvh: int, n: int, D: int, scale: float) -> torch.Tensor:
    """Rows 0..n of (block, kv head) from a flat view of a strided pool, as fp32 [n, D]."""
    flat = pool.reshape(-1)
    base = blk * strides[0] + kvh * strides[2]
    idx = base + torch.arange(n, device=pool.device)[:, None] * strides[1] + torch.arange(D, device=pool.device)[None, :]
    return _widen(flat[idx], scale)


# ----------------------------------------------------------------------------- tiled attention
def attn_state(num_seqs: int, Hq: int, D: int, device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Running state of a decode step before its first tile: m = -inf, l = o = 0."""
    m = torch.full((num_seqs, Hq), float("-inf"), dtype=torch.float32, device=device)
    return m, torch.zeros_like(m), torch.zeros(num_seqs, Hq, D, dtype=torch.float32, device=device)


def kv_tile_attn(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, tile_blocks: torch.Tensor,
                 tile_counts: torch.Tensor, state, *, Hkv: int, block_size: int, strides: Strides,
                 last_valid: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                 k_scale: float = 1.0, v_scale: float = 1.0, out: Optional[torch.Tensor] = None) -> None:
    """Fold one tile of KV blocks into ``state = (m, l, o)`` in place. ``q`` [S, Hq, D] bf16;
    ``tile_blocks`` [S, cap] int32 ids into the pools, ``tile_counts`` [S]; with ``last_valid`` only that
    many token slots of each sequence's last block of the tile are read. ``out`` (bf16 [S, Hq, D]), when
    given, receives o / l after this tile."""
    S, Hq, D = q.shape
    m, l, o = state
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if q.is_cuda:
        from ..ops import _count, _ptr, _stream
        a = KvTileArgs(_ptr(q.contiguous()), _ptr(k_pool), _ptr(v_pool), _ptr(tile_blocks), _ptr(tile_counts),
                       _ptr(last_valid), _ptr(m), _ptr(l), _ptr(o), _ptr(out), S, Hq, Hkv, D, block_size,
                       tile_blocks.shape[1], int(_is_fp8(k_pool)), strides[0], strides[1], strides[2],
                       scale, k_scale, v_scale)
        _native.check(_native.lib().mb_kv_tile_attn(C.byref(a), _stream()), f"kv_tile_attn[S={S} D={D}]")
        _count()
        return
    G = Hq // Hkv
    for s in range(S):
        nb = int(tile_counts[s])
        for b in range(nb):
            n = block_size
            if b == nb - 1 and last_valid is not None:
                n = max(0, min(block_size, int(last_valid[s])))
            if n == 0:
                continue
            blk = int(tile_blocks[s, b])
            for kh in range(Hkv):
                K = _rows(k_pool, strides, blk, kh, n, D, k_scale)
                V = _rows(v_pool, strides, blk, kh, n, D, v_scale)
                hs = slice(kh * G, (kh + 1) * G)
                sc = (q[s, hs].float() * scale) @ K.T                        # [G, n]
                mn = torch.maximum(m[s, hs], sc.max(dim=1).values)
                c_old = torch.where(torch.isinf(m[s, hs]), torch.zeros_like(mn), torch.exp(m[s, hs] - mn))
                p = torch.exp(sc - mn[:, None])
                l[s, hs] = l[s, hs] * c_old + p.sum(dim=1)
                o[s, hs] = o[s, hs] * c_old[:, None] + p @ V
                m[s, hs] = mn
    if out is not None:
        out.copy_(attn_finalize(l, o))


def attn_finalize(l: torch.Tensor, o: torch.Tensor) -> torch.Tensor:
    """o / l as bf16; rows that attended nothing (l == 0) are 0."""
    if o.is_cuda:
        from ..ops import _count, _ptr, _stream
        out = torch.empty(o.shape, dtype=torch.bfloat16, device=o.device)
        _native.check(_native.lib().mb_attn_finalize(_ptr(l), _ptr(o), _ptr(out), l.numel(), o.shape[-1], _stream()),
                      "attn_finalize")
        _count()
        return out
    safe = torch.where(l > 0, l, torch.ones_like(l))
    return torch.where((l > 0)[..., None], o / safe[..., None], torch.zeros_like(o)).to(torch.bfloat16)


# ----------------------------------------------------------------------------- predictor
def project_rows(x: torch.Tensor, P: torch.Tensor) -> torch.Tensor:
    """``x`` [..., D] bf16 times ``P`` [D, r] bf16 -> bf16 [..., r] (fp32 accumulation)."""
    D, r = P.shape
    if x.is_cuda:
        from ..ops import _count, _ptr, _stream
        xc = x.contiguous()
        out = torch.empty(*x.shape[:-1], r, dtype=torch.bfloat16, device=x.device)
        a = LowrankArgs(_ptr(xc), _ptr(P), _ptr(out), None, None, xc.numel() // D, D, r, 0, 0, 0, 0, 0, 0, 1.0)
        _native.check(_native.lib().mb_lowrank_project(C.byref(a), _stream()), f"lowrank_project[D={D} r={r}]")
        _count()
        return out
    return (x.float() @ P.float()).to(torch.bfloat16)


def project_blocks(k_pool: torch.Tensor, P: torch.Tensor, k_lr: torch.Tensor, src_blocks: torch.Tensor,
                   dst_blocks: torch.Tensor, *, Hkv: int, block_size: int, strides: Strides,
                   k_scale: float = 1.0) -> None:
    """Project every K row of pool blocks ``src_blocks`` and store them as ``k_lr[dst, kv_head, tok, :]``
    (``k_lr`` [blocks, Hkv, block, r] bf16): the layout ``predictor_score`` reads."""
    D, r = P.shape
    n = src_blocks.numel()
    if n == 0:
        return
    if k_pool.is_cuda:
        from ..ops import _count, _ptr, _stream
        a = LowrankArgs(_ptr(k_pool), _ptr(P), _ptr(k_lr), _ptr(src_blocks), _ptr(dst_blocks),
                        n * block_size * Hkv, D, r, Hkv, block_size, int(_is_fp8(k_pool)),
                        strides[0], strides[1], strides[2], k_scale)
        _native.check(_native.lib().mb_lowrank_project(C.byref(a), _stream()), f"lowrank_project[blocks={n}]")
        _count()
        return
    for j in range(n):
        for kh in range(Hkv):
            K = _rows(k_pool, strides, int(src_blocks[j]), kh, block_size, D, k_scale)
            k_lr[int(dst_blocks[j]), kh] = (K @ P.float()).to(torch.bfloat16)


def predictor_score(q_lr: torch.Tensor, k_lr: torch.Tensor, blocks: torch.Tensor, counts: torch.Tensor,
                    last_valid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``scores[s, b]`` = max over (query head, token) of <q_lr[s, head], k_lr[blocks[s, b], head / G, token]>;
    -inf past ``counts[s]``. ``q_lr`` [S, Hq, r], ``k_lr`` [blocks, Hkv, block, r], both bf16."""
    S, Hq, r = q_lr.shape
    _, Hkv, bs, _ = k_lr.shape
    cap = blocks.shape[1]
    if q_lr.is_cuda:
        from ..ops import _count, _ptr, _stream
        scores = torch.empty(S, cap, dtype=torch.float32, device=q_lr.device)
        a = ScoreArgs(_ptr(q_lr.contiguous()), _ptr(k_lr), _ptr(blocks), _ptr(counts), _ptr(last_valid),
                      _ptr(scores), S, Hq, Hkv, bs, r, cap)
        _native.check(_native.lib().mb_predictor_score(C.byref(a), _stream()), f"predictor_score[S={S} cap={cap}]")
        _count()
        return scores
    G = Hq // Hkv
    scores = torch.full((S, cap), float("-inf"), dtype=torch.float32)
    for s in range(S):
        nb = int(counts[s])
        for b in range(nb):
            n = bs
            if b == nb - 1 and last_valid is not None:
                n = max(0, min(bs, int(last_valid[s])))
            if n == 0:
                continue
            kb = k_lr[int(blocks[s, b]), :, :n].float()                                  # [Hkv, n, r]
            qg = q_lr[s].float().view(Hkv, G, r)
            scores[s, b] = torch.einsum("hgr,hnr->hgn", qg, kb).max()
    return scores
