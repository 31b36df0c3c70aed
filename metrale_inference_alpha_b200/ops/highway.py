"""Ops on the multi-stream fp32 residual highway of hyper-connection models (``csrc/hyperconn.cu``)
with their fp32 restatements: manifold-constrained hyper-connection pre / post, the engram gate, the
PLE gate and its dilated convolution, and the host-side n-gram hashing that feeds engram / PLE tables.

Reference: ``kernels/gb10/common/glm5next_mhc.cu``, ``kernels/gb10/deepseek-v4-flash/nvfp4/
{hyper_connection,engram_v41}.cu``, ``kernels/gb10/qwen3.8-flash-next/nvfp4/ple.cu``.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Sequence, Tuple

import torch

from . import _native

c_void_p, c_int, c_float = C.c_void_p, C.c_int, C.c_float

_native.register_optional("mb_hc_pre", [c_void_p] * 7 + [c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
_native.register_optional("mb_hc_pre_split", [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
_native.register_optional("mb_hc_post", [c_void_p] * 4 + [c_int, c_int, c_int, c_void_p])
_native.register_optional("mb_engram_gate_add", [c_void_p] * 3 + [c_int, c_int, c_int, c_float, c_void_p])
_native.register_optional("mb_ple_gate", [c_void_p] * 8 + [c_int, c_int, c_int, c_float, c_void_p])
_native.register_optional("mb_dilated_conv", [c_void_p] * 5 + [c_int, c_int, c_int] + [c_void_p] * 4 +
                          [c_int, c_int, c_int, c_void_p, c_void_p])


_HC_SPLIT_MIN_ROWS = 8


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and _native.available() and hasattr(_native.lib(), "mb_hc_pre")


def _ssqrt(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.sqrt(torch.clamp(x.abs(), min=1e-6))


# ----------------------------------------------------------------------------- hyper-connections
def hc_expand(x: torch.Tensor, hc: int) -> torch.Tensor:
    """Token embeddings [T, H] -> the highway [T, hc, H] fp32: every stream starts as the embedding."""
    return x.float()[:, None, :].expand(-1, hc, -1).contiguous()


def hc_head_mean(streams: torch.Tensor) -> torch.Tensor:
    """The highway collapsed for the final norm / LM head: the mean over streams, bf16 [T, H]."""
    return streams.mean(1).to(torch.bfloat16)


def hc_pre(streams: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, *, norm_eps: float = 1e-6,
           hc_eps: float = 1e-6, iters: int = 20) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``streams`` [T, hc, H] fp32, ``fn`` [(2 + hc) * hc, hc * H] bf16, ``scale`` [3], ``base`` [(2 + hc) * hc]
    fp32 -> (block input y bf16 [T, H], post [T, hc], comb [T, hc, hc])."""
    T, hc, H = streams.shape
    if _cuda(streams):
        from . import _count, _ptr, _stream
        y = torch.empty(T, H, dtype=torch.bfloat16, device=streams.device)
        post = torch.empty(T, hc, dtype=torch.float32, device=streams.device)
        comb = torch.empty(T, hc, hc, dtype=torch.float32, device=streams.device)
        L = _native.lib()
        if T >= _HC_SPLIT_MIN_ROWS and (hc * H) % 8 == 0 and hasattr(L, "mb_hc_pre_split"):
            # several rows: token tiles x slices of the stream axis, partial sums added in slice order
            L.mb_hc_pre_ws_floats.restype = c_int
            L.mb_hc_pre_ws_floats.argtypes = [c_int, c_int, c_int]
            need = int(L.mb_hc_pre_ws_floats(T, hc, H))
            ws = torch.empty(need, dtype=torch.float32, device=streams.device)
            rc = L.mb_hc_pre_split(_ptr(streams), _ptr(fn), _ptr(scale), _ptr(base), _ptr(y), _ptr(post), _ptr(comb), _ptr(ws),
                                   need, T, hc, H, norm_eps, hc_eps, iters, _stream())
            _native.check(rc, f"hc_pre_split[T={T}]")
            _count(2)
            return y, post, comb
        rc = _native.lib().mb_hc_pre(_ptr(streams), _ptr(fn), _ptr(scale), _ptr(base), _ptr(y), _ptr(post), _ptr(comb),
                                     T, hc, H, norm_eps, hc_eps, iters, _stream())
        _native.check(rc, f"hc_pre[T={T}]")
        _count()
        return y, post, comb
    flat = streams.reshape(T, hc * H).float()
    rstd = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + norm_eps)
    mix = (flat @ fn.float().T) * rstd
    pre = torch.sigmoid(mix[:, :hc] * scale[0] + base[:hc]) + hc_eps
    post = 2.0 * torch.sigmoid(mix[:, hc:2 * hc] * scale[1] + base[hc:2 * hc])
    comb = torch.softmax((mix[:, 2 * hc:] * scale[2] + base[2 * hc:]).view(T, hc, hc), -1) + hc_eps
    for it in range(iters):
        if it > 0:
            comb = comb / (comb.sum(2, keepdim=True) + hc_eps)
        comb = comb / (comb.sum(1, keepdim=True) + hc_eps)
    y = torch.einsum("ti,tid->td", pre, streams.float()).to(torch.bfloat16)
    return y, post, comb


def hc_post(block_out: torch.Tensor, streams: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """``streams[t, j] = post[t, j] * block_out[t] + sum_i comb[t, i, j] * streams[t, i]`` (in place on CUDA)."""
    T, hc, H = streams.shape
    if _cuda(streams):
        from . import _count, _ptr, _stream
        bo = block_out.to(torch.bfloat16).contiguous()
        rc = _native.lib().mb_hc_post(_ptr(bo), _ptr(streams), _ptr(post), _ptr(comb), T, hc, H, _stream())
        _native.check(rc, f"hc_post[T={T}]")
        _count()
        return streams
    bo = block_out.to(torch.bfloat16).float()
    streams.copy_(post[:, :, None] * bo[:, None, :] + torch.einsum("tij,tid->tjd", comb, streams.float()))
    return streams


# ----------------------------------------------------------------------------- engram / PLE
def ngram_hash_ids(tokens: Sequence[int], n: int, table_rows: int, cols: int, seed: int = 0x9E3779B1) -> List[List[int]]:
    """Row ids of the hashed n-gram table for every position: ``cols`` independent multiplicative hashes of
    the last ``n`` token ids ending at the position (shorter windows at the start). Computed on the host:
    the ids select rows of a table that may live behind a file-backed row cache."""
    out = []
    for t in range(len(tokens)):
        win = tokens[max(0, t - n + 1):t + 1]
        row = []
        for c in range(cols):
            h = (seed + 0x85EBCA77 * (c + 1)) & 0xFFFFFFFF
            for tok in win:
                h = ((h ^ (int(tok) + 0x165667B1)) * 0x9E3779B1) & 0xFFFFFFFF
                h ^= h >> 15
            row.append(h % table_rows)
        out.append(row)
    return out


def engram_gate_add(streams: torch.Tensor, kv: torch.Tensor, qk: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``streams`` [T, hc, H] fp32 += sigmoid(ssqrt(dot)) * value, per stream; ``kv`` [T, (hc + 1) * H] bf16 =
    the hc keys then the shared value, ``qk`` [hc, H] fp32 = the product of the query and key norm weights."""
    T, hc, H = streams.shape
    if _cuda(streams):
        from . import _count, _ptr, _stream
        rc = _native.lib().mb_engram_gate_add(_ptr(streams), _ptr(kv.contiguous()), _ptr(qk), T, hc, H, eps, _stream())
        _native.check(rc, f"engram_gate_add[T={T}]")
        _count()
        return streams
    key = kv[:, :hc * H].float().view(T, hc, H)
    val = kv[:, hc * H:].float()
    h = streams.float()
    rstd = torch.rsqrt(h.pow(2).mean(-1) + eps) * torch.rsqrt(key.pow(2).mean(-1) + eps)
    dot = (h * qk[None] * key).sum(-1) * rstd / math.sqrt(H)
    streams.add_(torch.sigmoid(_ssqrt(dot))[..., None] * val[:, None, :])
    return streams


def ple_gate(hidden: torch.Tensor, key: torch.Tensor, value: torch.Tensor, w_key: torch.Tensor, w_query: torch.Tensor,
             w_conv: torch.Tensor, eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """``hidden`` [T, hc, H] fp32 highway, ``key`` [T, hc * H] bf16, ``value`` [T, H] bf16; the three norm
    weights [hc, H] are applied as (1 + w) over each stream's own slice. Returns (gated [T, hc * H] fp32,
    its grouped RMSNorm for the convolution)."""
    T, hc, H = hidden.shape
    if _cuda(hidden):
        from . import _count, _ptr, _stream
        gated = torch.empty(T, hc * H, dtype=torch.float32, device=hidden.device)
        normed = torch.empty_like(gated)
        rc = _native.lib().mb_ple_gate(_ptr(hidden), _ptr(key.contiguous()), _ptr(value.contiguous()), _ptr(w_key),
                                       _ptr(w_query), _ptr(w_conv), _ptr(gated), _ptr(normed), T, hc, H, eps, _stream())
        _native.check(rc, f"ple_gate[T={T}]")
        _count()
        return gated, normed
    rms = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w)
    kn = rms(key.float().view(T, hc, H), w_key)
    qn = rms(hidden.float(), w_query)
    g = torch.sigmoid(_ssqrt((kn * qn).sum(-1) / math.sqrt(H)))
    gated = g[..., None] * value.float()[:, None, :]
    return gated.reshape(T, hc * H), rms(gated, w_conv).reshape(T, hc * H)


def dilated_conv(x: torch.Tensor, base: torch.Tensor, w: torch.Tensor, state: torch.Tensor, batch, dilation: int,
                 write_state: bool = True) -> torch.Tensor:
    """``base + silu(depthwise causal conv of x with taps w [C, taps] at the given dilation)`` over a ragged
    batch; ``state`` [slots, C, (taps - 1) * dilation] fp32 carries the inputs before each sequence's rows."""
    T, Cn = x.shape
    taps = w.shape[1]
    hist = (taps - 1) * dilation
    if _cuda(x):
        from . import _count, _ptr, _stream, runtime
        out = torch.empty_like(x)
        rc = _native.lib().mb_dilated_conv(_ptr(x.contiguous()), _ptr(base.contiguous()), _ptr(w), _ptr(state), _ptr(out),
                                           Cn, taps, dilation, _ptr(batch.q_start), _ptr(batch.q_len),
                                           _ptr(batch.positions), _ptr(batch.state_slots), batch.q_len.numel(),
                                           state.shape[0], int(write_state), _ptr(runtime(x.device).status), _stream())
        _native.check(rc, f"dilated_conv[T={T}]")
        _count()
        return out
    out = torch.empty_like(x)
    qs, ql = batch.q_start.tolist(), batch.q_len.tolist()
    for s, n in enumerate(ql):
        if n <= 0:
            continue
        q0, slot = qs[s], int(batch.state_slots[s])
        old = torch.zeros(Cn, hist) if int(batch.positions[q0]) == 0 else state[slot].clone()
        full = torch.cat([old.T, x[q0:q0 + n].float()], 0)                       # [hist + n, C]
        for t in range(n):
            acc = sum(w[:, j] * full[hist + t - (taps - 1 - j) * dilation] for j in range(taps))
            out[q0 + t] = base[q0 + t] + torch.nn.functional.silu(acc)
        if write_state:
            state[slot] = full[-hist:].T
    return out
