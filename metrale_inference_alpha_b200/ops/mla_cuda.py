"""Binding of the absorbed-MLA paged attention kernel (``csrc/mla.cu``): multi-query attention of
``[T, H, 576]`` absorbed queries over the latent cache ``[blocks, block, 1, 576]`` (bf16), values =
the first 512 dims of each cached row. On CPU tensors the fp32 restatement in ``models/mla.py`` runs."""
from __future__ import annotations

import ctypes as C

import torch

from . import _native

c_void_p, c_int, c_ll, c_float, c_size_t = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_size_t


class MlaArgs(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("cache", c_void_p), ("block_table", c_void_p), ("max_blocks", c_int),
        ("q_start", c_void_p), ("q_len", c_void_p), ("ctx_len", c_void_p), ("row_seq", c_void_p),
        ("num_seqs", c_int), ("max_q_len", c_int), ("max_ctx", c_int), ("total_rows", c_int),
        ("H", c_int), ("block_size", c_int), ("num_blocks", c_ll), ("scale", c_float),
        ("out", c_void_p), ("ws", c_void_p), ("ws_bytes", c_size_t), ("part_tokens", c_int), ("status", c_void_p),
        ("impl", c_int),
    ]


_native.register_optional("mb_mla_attention", [C.POINTER(MlaArgs), c_void_p])

_native.register_optional("mb_mla_prepare", [c_void_p] * 10 + [c_int] * 6 + [c_ll, c_float, c_void_p, c_void_p])

LATENT, ROW = 512, 576
TC_PART_TOKENS = 256
_CNT_BYTES = 64 * 1024


def supported(q: torch.Tensor, cache: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and q.shape[-1] == ROW
            and cache.shape[-1] == ROW and cache.shape[2] == 1)


def mla_attention(q: torch.Tensor, cache: torch.Tensor, block_table, q_start, q_len, ctx_len, *, max_q_len: int,
                  max_ctx: int, scale: float, row_seq=None, part_tokens: int = 0, impl: int = 0) -> torch.Tensor:
    """q [T, H, 576] bf16 -> [T, H, 512] fp32. `impl`: 0 = decode steps (one query row per sequence,
    16 <= H <= 128) take the tcgen05 / TMEM kernel, everything else the mma.sync kernel; 1 / 2 force one."""
    from . import _count, _ptr, _stream, runtime
    L = _native.lib()
    if not hasattr(L, "mb_mla_attention"):
        raise RuntimeError("kernel library was built without mla.cu")
    L.mb_mla_ws_bytes.argtypes = [c_int, c_int, c_int, c_int]
    L.mb_mla_ws_bytes.restype = c_size_t
    T, H, _ = q.shape
    q = q.contiguous()
    if part_tokens == 0 and impl != 1 and max_q_len == 1 and 16 <= H <= 128:
        # the tcgen05 decode kernel runs one CTA per SM: shorter partitions than the mma.sync kernel's 1024
        # keep the SMs busy at small batch (a constant, so a sequence's split never depends on the batch)
        part_tokens = TC_PART_TOKENS
    rt = runtime(q.device)
    out = torch.empty(T, H, LATENT, dtype=torch.float32, device=q.device)
    need = L.mb_mla_ws_bytes(T, H, max_ctx, part_tokens)
    if need:
        # the head of the shared attention workspace holds the split-KV kernel's arrival counters,
        # which must stay zero between its launches: the MLA partials live behind them
        rt.ensure_attn_ws(need + _CNT_BYTES)
        if row_seq is None:                       # row -> sequence map for the merge pass
            # fixed-shape (capturable): the sequence of row t is the last one whose first row is <= t
            rows = torch.arange(T, device=q.device, dtype=q_start.dtype)
            row_seq = (torch.bucketize(rows, q_start, right=True) - 1).clamp(min=0).to(torch.int32).contiguous()
    a = MlaArgs()
    a.q, a.cache, a.block_table, a.max_blocks = _ptr(q), _ptr(cache), _ptr(block_table), block_table.stride(0)
    a.q_start, a.q_len, a.ctx_len, a.row_seq = _ptr(q_start), _ptr(q_len), _ptr(ctx_len), _ptr(row_seq)
    a.num_seqs, a.max_q_len, a.max_ctx, a.total_rows = q_len.numel(), max_q_len, max_ctx, T
    a.H, a.block_size, a.num_blocks, a.scale = H, cache.shape[1], cache.shape[0], scale
    a.out, a.part_tokens, a.status, a.impl = _ptr(out), part_tokens, _ptr(rt.status), impl
    a.ws, a.ws_bytes = (_ptr(rt.attn_ws) + _CNT_BYTES, rt.attn_ws.numel() - _CNT_BYTES) if need else (None, 0)
    _native.check(L.mb_mla_attention(C.byref(a), _stream()), "mla_attention")
    _count()
    return out


def prepare(q: torch.Tensor, q_lat: torch.Tensor, ckv: torch.Tensor, norm_w: torch.Tensor, cos, sin, positions,
            slots, cache: torch.Tensor, nope: int, eps: float) -> torch.Tensor:
    """One launch: latent RMSNorm + key RoPE + cache row write, and the absorbed query rows
    [T, H, L + R] assembled from q_lat [H, T, L] and the rotated rope part of q [T, H, nope + R]."""
    from . import _count, _ptr, _stream, runtime
    T, H, qd = q.shape
    L, R = q_lat.shape[-1], qd - nope
    qq = torch.empty(T, H, L + R, dtype=torch.bfloat16, device=q.device)
    rc = _native.lib().mb_mla_prepare(
        _ptr(q), _ptr(q_lat), _ptr(ckv), _ptr(norm_w), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots),
        _ptr(cache), _ptr(qq), T, H, nope, R, L, cos.shape[0], cache.shape[0] * cache.shape[1], eps,
        _ptr(runtime(q.device).status), _stream())
    _native.check(rc, "mla_prepare")
    _count()
    return qq
