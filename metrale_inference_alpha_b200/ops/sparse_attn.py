"""Sparse (indexed) attention ops: indexer scores, deterministic top-k selection, gather of the selected
cache rows, and latent attention over the selection (``csrc/sparse_index.cu`` + the dense MLA kernel
over the gathered rows). CPU tensors take the fp32 restatements below, which are also the oracles of
the GPU tests.

Reference: ``kernels/gb10/common/dsa_indexer.cu`` (score -> top-k -> expand -> compact) and
``glm5next_dsa_mla_decode.cu``.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import torch

from . import _native

c_void_p, c_int, c_ll = C.c_void_p, C.c_int, C.c_longlong

_native.register_optional("mb_index_score", [c_void_p] * 4 + [c_int] + [c_void_p] * 3 + [c_ll, c_int, c_int, c_int, c_int, c_ll,
                                                                                    c_void_p, c_void_p])
_native.register_optional("mb_topk_select", [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
_native.register_optional("mb_gather_rows", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_int, c_int, c_int, c_ll, c_void_p, c_void_p])


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and _native.available() and hasattr(_native.lib(), "mb_index_score")


def row_meta(batch) -> Tuple[torch.Tensor, torch.Tensor]:
    """(sequence of every token row, number of tokens the row sees = its position + 1), both int32."""
    S = batch.q_len.numel()
    seq = torch.repeat_interleave(torch.arange(S, dtype=torch.int32, device=batch.q_len.device), batch.q_len.long(),
                                  output_size=batch.positions.numel())
    return seq, (batch.positions + 1).to(torch.int32)


def index_scores(iq: torch.Tensor, iw: torch.Tensor, kcache: torch.Tensor, block_table: torch.Tensor,
                 row_seq: torch.Tensor, row_ctx: torch.Tensor, max_ctx: int) -> torch.Tensor:
    """``iq`` [T, Hi, Di] bf16, ``iw`` [T, Hi] fp32, ``kcache`` [blocks, block, 1, Di] bf16 ->
    fp32 [T, ld] with ld = max_ctx rounded up to 64; -inf at and past ``row_ctx[t]``."""
    T, Hi, Di = iq.shape
    nb, bs = kcache.shape[0], kcache.shape[1]
    ld = (max_ctx + 63) // 64 * 64
    if _cuda(iq):
        from . import _count, _ptr, _stream, runtime
        scores = torch.empty(T, ld, dtype=torch.float32, device=iq.device)
        rc = _native.lib().mb_index_score(_ptr(iq.contiguous()), _ptr(iw.contiguous()), _ptr(kcache), _ptr(block_table),
                                          block_table.shape[1], _ptr(row_seq), _ptr(row_ctx), _ptr(scores), ld, T, Hi, Di,
                                          bs, nb, _ptr(runtime(iq.device).status), _stream())
        _native.check(rc, f"index_score[T={T} ctx={max_ctx}]")
        _count()
        return scores
    scores = torch.full((T, ld), float("-inf"), dtype=torch.float32)
    flat = kcache.reshape(nb * bs, Di).float()
    for t in range(T):
        n = int(row_ctx[t])
        if n <= 0:
            continue
        pos = torch.arange(n)
        rows = flat[block_table[int(row_seq[t]), pos // bs].long() * bs + pos % bs]            # [n, Di]
        dots = torch.relu(iq[t].float() @ rows.T)                                              # [Hi, n]
        scores[t, :n] = (iw[t].float()[:, None] * dots).sum(0)
    return scores


def topk_indices(scores: torch.Tensor, row_ctx: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per row the positions of the k largest scores among the first ``row_ctx[t]`` (ties to the lower
    position), ascending, padded with -1; rows that see at most k tokens select all of them. Returns
    (idx [T, k] int32, count [T] int32)."""
    T = scores.shape[0]
    if _cuda(scores):
        from . import _count, _ptr, _stream
        idx = torch.empty(T, k, dtype=torch.int32, device=scores.device)
        cnt = torch.empty(T, dtype=torch.int32, device=scores.device)
        rc = _native.lib().mb_topk_select(_ptr(scores), scores.stride(0), _ptr(row_ctx), T, k, _ptr(idx), _ptr(cnt), _stream())
        _native.check(rc, f"topk_select[T={T} k={k}]")
        _count()
        return idx, cnt
    idx = torch.full((T, k), -1, dtype=torch.int32)
    cnt = torch.zeros(T, dtype=torch.int32)
    for t in range(T):
        n = max(0, int(row_ctx[t]))
        if n <= k:
            idx[t, :n] = torch.arange(n, dtype=torch.int32)
            cnt[t] = n
        else:
            order = torch.sort(scores[t, :n], descending=True, stable=True).indices[:k]        # stable: ties keep position order
            idx[t] = torch.sort(order).values.to(torch.int32)
            cnt[t] = k
    return idx, cnt


def gather_rows(cache: torch.Tensor, block_table: torch.Tensor, row_seq: torch.Tensor, idx: torch.Tensor,
                count: torch.Tensor) -> torch.Tensor:
    """The selected tokens' cache rows as a compact paged buffer ``[T * kb, block, 1, W]`` (kb = k rounded
    up to whole blocks): row t owns blocks t*kb .. (t+1)*kb, its j-th selected token sits at slot j."""
    nb, bs, _, W = cache.shape
    T, k = idx.shape
    kb = (k + bs - 1) // bs
    if _cuda(cache):
        from . import _count, _ptr, _stream, runtime
        dst = torch.empty(T * kb, bs, 1, W, dtype=cache.dtype, device=cache.device)
        rc = _native.lib().mb_gather_rows(_ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(row_seq), _ptr(idx),
                                          _ptr(count), _ptr(dst), T, k, kb * bs, W * cache.element_size(), bs, nb,
                                          _ptr(runtime(cache.device).status), _stream())
        _native.check(rc, f"gather_rows[T={T} k={k}]")
        _count()
        return dst
    dst = torch.zeros(T, kb * bs, W, dtype=cache.dtype)
    flat = cache.reshape(nb * bs, W)
    for t in range(T):
        n = int(count[t])
        if n:
            tok = idx[t, :n].long()
            dst[t, :n] = flat[block_table[int(row_seq[t]), tok // bs].long() * bs + tok % bs]
    return dst.view(T * kb, bs, 1, W)


def selected_latent_attention(qq: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, row_seq: torch.Tensor,
                              idx: torch.Tensor, count: torch.Tensor, scale: float, latent: int) -> torch.Tensor:
    """Latent (MLA) attention of every query row over its own selected tokens: ``qq`` [T, H, W] bf16 ->
    fp32 [T, H, latent]. The selection is gathered into a compact buffer and each row runs as a
    one-token sequence over it."""
    T, H, W = qq.shape
    bs = cache.shape[1]
    compact = gather_rows(cache, block_table, row_seq, idx, count)
    kb = compact.shape[0] // T
    dev = qq.device
    from . import mla_cuda
    if qq.is_cuda and mla_cuda.supported(qq, compact) and latent == mla_cuda.LATENT:
        tbl = torch.arange(T * kb, dtype=torch.int32, device=dev).view(T, kb)
        ones = torch.ones(T, dtype=torch.int32, device=dev)
        return mla_cuda.mla_attention(qq, compact, tbl, torch.arange(T, dtype=torch.int32, device=dev), ones, count,
                                      max_q_len=1, max_ctx=kb * bs, scale=scale)
    rows = compact.view(T, kb * bs, W).float()
    out = torch.zeros(T, H, latent, dtype=torch.float32, device=dev)
    for t in range(T):
        n = int(count[t])
        if n:
            sc = (qq[t].float() @ rows[t, :n].T) * scale
            out[t] = torch.softmax(sc, -1) @ rows[t, :n, :latent]
    return out
