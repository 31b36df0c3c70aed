"""Recurrent-state ops over a ragged batch: causal conv1d with a carried window,
gated-delta-net recurrence, Mamba2 selective scan. CUDA tensors run the kernels in
``csrc/recurrent.cu``; CPU tensors run the reference loops (the oracle).

State tensors are indexed by ``batch.state_slots[s]``; a sequence whose first row is at
position 0 starts from a zero state.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native, reference as ref
from . import _count, _ptr, _stream


def _seq_rows(batch):
    qs, ql = batch.q_start.tolist(), batch.q_len.tolist()
    slots = batch.state_slots.tolist()
    pos0 = [int(batch.positions[qs[s]]) if ql[s] > 0 else 0 for s in range(len(ql))]
    return qs, ql, slots, pos0


def causal_conv1d(x: torch.Tensor, channels: int, w: torch.Tensor, bias, state: torch.Tensor, batch,
                  activation: bool = True, write_state: bool = True, write_out: bool = True) -> torch.Tensor:
    """x [T, >=channels] (first `channels` columns are convolved), w [C, taps] (tap 0 oldest),
    state [slots, C, taps-1] fp32. Returns fp32 [T, C]; updates the window in place.
    `write_state=False` leaves the state untouched (speculative verification);
    `write_out=False` only advances the state (the commit pass over the accepted tokens).
    The same two switches exist on the two recurrences below."""
    if x.is_cuda and _native.available() and hasattr(_native.lib(), "mb_causal_conv1d"):
        return _conv_cuda(x, channels, w, bias, state, batch, activation, write_state, write_out)
    T = x.shape[0]
    out = torch.empty(T, channels, dtype=torch.float32, device=x.device)
    qs, ql, slots, pos0 = _seq_rows(batch)
    for s in range(len(ql)):
        if slots[s] == 0 and False:
            continue
        st = state[slots[s]:slots[s] + 1]
        if pos0[s] == 0:
            st = torch.zeros_like(st)
        for t in range(qs[s], qs[s] + ql[s]):
            y, st = ref.causal_conv1d_update(st, x[t:t + 1, :channels], w, bias, activation)
            out[t] = y[0]
        if write_state and ql[s] > 0:
            state[slots[s]] = st[0]
    return out


def gdn_recurrence(conv_out, ba, A_log, dt_bias, state, batch, *, k_heads, v_heads, k_dim, v_dim,
                   write_state: bool = True, write_out: bool = True):
    """conv_out [T, 2 QK + V] fp32 (q | k | v after conv + SiLU), ba [T, 2 v_heads] fp32
    (b | a). Applies l2-norm to q and k per head, computes decay/beta, runs the delta rule.
    state [slots, v_heads, k_dim, v_dim] fp32. Returns fp32 [T, v_heads * v_dim]."""
    if conv_out.is_cuda and _native.available() and hasattr(_native.lib(), "mb_gdn_recurrence"):
        if (write_out and k_dim == 128 and v_dim == 128 and getattr(batch, "max_q_len", 1) >= _GDN_CHUNK_MIN_TOKENS
                and hasattr(_native.lib(), "mb_gdn_chunked")):
            y = _gdn_chunked_cuda(conv_out, ba, A_log, dt_bias, state, batch, k_heads, v_heads, write_state)
            if y is not None:
                return y
        return _gdn_cuda(conv_out, ba, A_log, dt_bias, state, batch, k_heads, v_heads, k_dim, v_dim, write_state, write_out)
    T = conv_out.shape[0]
    QK, V = k_heads * k_dim, v_heads * v_dim
    out = torch.empty(T, V, dtype=torch.float32, device=conv_out.device)
    qs, ql, slots, pos0 = _seq_rows(batch)
    decay, beta = ref.gdn_gates(ba[:, v_heads:], ba[:, :v_heads], A_log, dt_bias)
    for s in range(len(ql)):
        h = state[slots[s]:slots[s] + 1].clone()
        if pos0[s] == 0:
            h.zero_()
        for t in range(qs[s], qs[s] + ql[s]):
            q = ref.l2_norm(conv_out[t, :QK].view(1, k_heads, k_dim))
            k = ref.l2_norm(conv_out[t, QK:2 * QK].view(1, k_heads, k_dim))
            v = conv_out[t, 2 * QK:2 * QK + V].view(1, v_heads, v_dim)
            o, h = ref.gdn_recurrence_step(h, q, k, v, decay[t:t + 1], beta[t:t + 1])
            out[t] = o.reshape(-1)
        if write_state and ql[s] > 0:
            state[slots[s]] = h[0]
    return out


def mamba2_scan(xbc, dt, A_log, D, dt_bias, ssm_state, batch, *, heads, groups, head_dim, state,
                write_state: bool = True, write_out: bool = True):
    """xbc [T, inner + 2 G N] fp32 (x | B | C after conv + SiLU), dt [T, heads] (raw).
    ssm_state [slots, heads, head_dim, state] fp32. Returns fp32 [T, heads * head_dim]."""
    if xbc.is_cuda and _native.available() and hasattr(_native.lib(), "mb_mamba2_scan"):
        if (write_out and head_dim == 64 and state == 128 and getattr(batch, "max_q_len", 1) >= _SSD_MIN_TOKENS
                and hasattr(_native.lib(), "mb_mamba2_ssd")):
            y = _mamba_ssd_cuda(xbc, dt, A_log, D, dt_bias, ssm_state, batch, heads, groups, write_state)
            if y is not None:
                return y
        return _mamba_cuda(xbc, dt, A_log, D, dt_bias, ssm_state, batch, heads, groups, head_dim, state, write_state, write_out)
    T = xbc.shape[0]
    inner, GN = heads * head_dim, groups * state
    out = torch.empty(T, inner, dtype=torch.float32, device=xbc.device)
    qs, ql, slots, pos0 = _seq_rows(batch)
    for s in range(len(ql)):
        h = ssm_state[slots[s]:slots[s] + 1].clone()
        if pos0[s] == 0:
            h.zero_()
        for t in range(qs[s], qs[s] + ql[s]):
            x = xbc[t, :inner].view(1, heads, head_dim)
            B = xbc[t, inner:inner + GN].view(1, groups, state)
            Cm = xbc[t, inner + GN:inner + 2 * GN].view(1, groups, state)
            y, h = ref.mamba2_step(h, x, dt[t:t + 1].float(), A_log, B, Cm, D, dt_bias)
            out[t] = y.reshape(-1)
        if write_state and ql[s] > 0:
            ssm_state[slots[s]] = h[0]
    return out


# ----------------------------------------------------------------------------- CUDA launchers
_c = C
_native.register_optional("mb_causal_conv1d", [_c.c_void_p, _c.c_longlong, _c.c_int, _c.c_int, _c.c_void_p,
                                              _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                              _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                              _c.c_void_p, _c.c_void_p])
_native.register_optional("mb_gdn_recurrence", [_c.c_void_p] * 6 + [_c.c_int] * 4 + [_c.c_void_p] * 4 +
                          [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p])
_native.register_optional("mb_mamba2_scan", [_c.c_void_p, _c.c_void_p, _c.c_longlong] + [_c.c_void_p] * 5 +
                          [_c.c_int] * 4 + [_c.c_void_p] * 4 + [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p])


_native.register_optional("mb_mamba2_ssd", [_c.c_void_p, _c.c_void_p, _c.c_longlong] + [_c.c_void_p] * 5 +
                          [_c.c_int] * 4 + [_c.c_void_p] * 4 + [_c.c_int] * 4 + [_c.c_void_p, _c.c_size_t, _c.c_void_p,
                                                                                _c.c_void_p])
# prefill chunks at least this long take the chunked (state-space-dual) Mamba2 scan
_SSD_MIN_TOKENS = 32
_SSD_WS_MAX = 3 << 30
_ssd_ws = {}


def _mamba_ssd_cuda(xbc, dt, A_log, D, dt_bias, ssm_state, batch, heads, groups, write_state):
    """Chunked scan (csrc/recurrent_chunked.cu); None when the workspace would be unreasonably large."""
    L = _native.lib()
    L.mb_mamba2_ssd_ws_bytes.restype = _c.c_size_t
    L.mb_mamba2_ssd_ws_bytes.argtypes = [_c.c_int, _c.c_int, _c.c_int]
    S = batch.q_len.numel()
    need = int(L.mb_mamba2_ssd_ws_bytes(S, int(batch.max_q_len), heads))
    if need > _SSD_WS_MAX:
        return None
    dev = xbc.device
    ws = _ssd_ws.get(dev)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            return None
        ws = _ssd_ws[dev] = torch.empty(int(need * 1.25), dtype=torch.uint8, device=dev)
    T = xbc.shape[0]
    out = torch.empty(T, heads * 64, dtype=torch.float32, device=dev)
    assert dt.dtype == torch.bfloat16
    rc = L.mb_mamba2_ssd(
        _ptr(xbc), _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(D), _ptr(dt_bias), _ptr(ssm_state), _ptr(out),
        heads, groups, 64, 128, _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions),
        _ptr(batch.state_slots), S, ssm_state.shape[0], int(batch.max_q_len), int(write_state), _ptr(ws), ws.numel(),
        _ptr(_status(dev)), _stream())
    _native.check(rc, "mamba2_ssd")
    _count(3)
    return out


_native.register_optional("mb_gdn_chunked", [_c.c_void_p] * 6 + [_c.c_int] * 4 + [_c.c_void_p] * 4 + [_c.c_int] * 4 +
                          [_c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p])
# prefill chunks at least this long take the chunked gated delta rule
_GDN_CHUNK_MIN_TOKENS = 64
_gdn_ws = {}


def _gdn_chunked_cuda(conv_out, ba, A_log, dt_bias, state, batch, k_heads, v_heads, write_state):
    """Chunked delta rule (csrc/gdn_chunked.cu); None when the workspace would be unreasonably large."""
    L = _native.lib()
    L.mb_gdn_chunked_ws_bytes.restype = _c.c_size_t
    L.mb_gdn_chunked_ws_bytes.argtypes = [_c.c_int, _c.c_int, _c.c_int]
    S = batch.q_len.numel()
    need = int(L.mb_gdn_chunked_ws_bytes(S, int(batch.max_q_len), v_heads))
    if need > _SSD_WS_MAX:
        return None
    dev = conv_out.device
    ws = _gdn_ws.get(dev)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            return None
        ws = _gdn_ws[dev] = torch.empty(int(need * 1.25), dtype=torch.uint8, device=dev)
    T = conv_out.shape[0]
    out = torch.empty(T, v_heads * 128, dtype=torch.float32, device=dev)
    rc = L.mb_gdn_chunked(
        _ptr(conv_out), _ptr(ba), _ptr(A_log), _ptr(dt_bias), _ptr(state), _ptr(out), k_heads, v_heads, 128, 128,
        _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions), _ptr(batch.state_slots), S, state.shape[0],
        int(batch.max_q_len), int(write_state), _ptr(ws), ws.numel(), _ptr(_status(dev)), _stream())
    _native.check(rc, "gdn_chunked")
    _count(2)
    return out


def _status(dev):
    from . import runtime
    return runtime(dev).status


_native.register_optional("mb_causal_conv1d_par", [_c.c_void_p, _c.c_longlong, _c.c_int, _c.c_int, _c.c_void_p,
                                                  _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                                  _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                                  _c.c_void_p, _c.c_void_p])
# prefill chunks at least this long take the time-parallel convolution
_CONV_PAR_MIN_TOKENS = 64


def _conv_cuda(x, channels, w, bias, state, batch, activation, write_state=True, write_out=True):
    T = x.shape[0]
    out = torch.empty(T, channels, dtype=torch.float32, device=x.device)
    mq = int(getattr(batch, "max_q_len", 1))
    if write_out and mq >= _CONV_PAR_MIN_TOKENS and hasattr(_native.lib(), "mb_causal_conv1d_par"):
        rc = _native.lib().mb_causal_conv1d_par(
            _ptr(x), x.stride(0), channels, w.shape[1], _ptr(w), _ptr(bias), _ptr(state), _ptr(out),
            _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions), _ptr(batch.state_slots),
            batch.q_len.numel(), state.shape[0], mq, int(activation), int(write_state), _ptr(_status(x.device)), _stream())
        _native.check(rc, "causal_conv1d_par")
        _count(2 if write_state else 1)
        return out
    rc = _native.lib().mb_causal_conv1d(
        _ptr(x), x.stride(0), channels, w.shape[1], _ptr(w), _ptr(bias), _ptr(state), _ptr(out),
        _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions), _ptr(batch.state_slots),
        batch.q_len.numel(), state.shape[0], int(activation), int(write_state), int(write_out),
        _ptr(_status(x.device)), _stream())
    _native.check(rc, "causal_conv1d")
    _count()
    return out


def _gdn_cuda(conv_out, ba, A_log, dt_bias, state, batch, k_heads, v_heads, k_dim, v_dim, write_state=True, write_out=True):
    T = conv_out.shape[0]
    out = torch.empty(T, v_heads * v_dim, dtype=torch.float32, device=conv_out.device)
    rc = _native.lib().mb_gdn_recurrence(
        _ptr(conv_out), _ptr(ba), _ptr(A_log), _ptr(dt_bias), _ptr(state), _ptr(out), k_heads, v_heads,
        k_dim, v_dim, _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions),
        _ptr(batch.state_slots), batch.q_len.numel(), state.shape[0], int(write_state), int(write_out),
        _ptr(_status(conv_out.device)), _stream())
    _native.check(rc, "gdn_recurrence")
    _count()
    return out


def _mamba_cuda(xbc, dt, A_log, D, dt_bias, ssm_state, batch, heads, groups, head_dim, state, write_state=True, write_out=True):
    T = xbc.shape[0]
    out = torch.empty(T, heads * head_dim, dtype=torch.float32, device=xbc.device)
    assert dt.dtype == torch.bfloat16
    rc = _native.lib().mb_mamba2_scan(
        _ptr(xbc), _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(D), _ptr(dt_bias), _ptr(ssm_state), _ptr(out),
        heads, groups, head_dim, state, _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions),
        _ptr(batch.state_slots), batch.q_len.numel(), ssm_state.shape[0], int(write_state), int(write_out),
        _ptr(_status(xbc.device)), _stream())
    _native.check(rc, "mamba2_scan")
    _count()
    return out


# ----------------------------------------------------------------------------- Kimi delta attention
import ctypes as _C


class _KdaArgs(_C.Structure):
    _fields_ = [("conv", _C.c_void_p), ("g_raw", _C.c_void_p), ("b_raw", _C.c_void_p), ("b_ld", _C.c_int),
                ("A_log", _C.c_void_p), ("dt_bias", _C.c_void_p), ("lower_bound", _C.c_float), ("state", _C.c_void_p),
                ("out", _C.c_void_p), ("out_norm", _C.c_void_p), ("out_gate", _C.c_void_p), ("gate_ld", _C.c_longlong),
                ("norm_w", _C.c_void_p), ("eps", _C.c_float), ("H", _C.c_int), ("D", _C.c_int),
                ("q_start", _C.c_void_p), ("q_len", _C.c_void_p), ("positions", _C.c_void_p),
                ("state_slots", _C.c_void_p), ("num_seqs", _C.c_int), ("num_slots", _C.c_int),
                ("write_state", _C.c_int), ("write_out", _C.c_int), ("status", _C.c_void_p)]


_native.register_optional("mb_kda_recurrence", [_C.POINTER(_KdaArgs), _C.c_void_p])


_KDA_CHUNK_MIN_TOKENS = 64
_kda_ws: dict = {}


class _KdaChunkedArgs(_C.Structure):
    _fields_ = [("conv", _C.c_void_p), ("g_raw", _C.c_void_p), ("b_raw", _C.c_void_p), ("b_ld", _C.c_int),
                ("A_log", _C.c_void_p), ("dt_bias", _C.c_void_p), ("lower_bound", _C.c_float), ("state", _C.c_void_p),
                ("out", _C.c_void_p), ("out_norm", _C.c_void_p), ("out_gate", _C.c_void_p), ("gate_ld", _C.c_longlong),
                ("norm_w", _C.c_void_p), ("eps", _C.c_float), ("H", _C.c_int), ("D", _C.c_int),
                ("q_start", _C.c_void_p), ("q_len", _C.c_void_p), ("positions", _C.c_void_p),
                ("state_slots", _C.c_void_p), ("num_seqs", _C.c_int), ("num_slots", _C.c_int), ("max_q_len", _C.c_int),
                ("total_rows", _C.c_int), ("write_state", _C.c_int), ("ws", _C.c_void_p), ("ws_bytes", _C.c_size_t),
                ("status", _C.c_void_p)]


_native.register_optional("mb_kda_chunked", [_C.POINTER(_KdaChunkedArgs), _C.c_void_p])


def _kda_chunked_cuda(conv_out, g_raw, b_raw, A_log, dt_bias, lower_bound, state, batch, H, write_state, norm):
    """Chunked prefill (csrc/kda_chunked.cu); None when the workspace would be unreasonably large."""
    L = _native.lib()
    L.mb_kda_chunked_ws_bytes.restype = _C.c_size_t
    L.mb_kda_chunked_ws_bytes.argtypes = [_C.c_int, _C.c_int, _C.c_int]
    S = batch.q_len.numel()
    need = int(L.mb_kda_chunked_ws_bytes(S, int(batch.max_q_len), H))
    if need > _SSD_WS_MAX:
        return None
    dev = conv_out.device
    ws = _kda_ws.get(dev)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            return None
        ws = _kda_ws[dev] = torch.empty(int(need * 1.25), dtype=torch.uint8, device=dev)
    T = conv_out.shape[0]
    out = torch.empty(T, H * 128, dtype=torch.float32, device=dev)
    out_n = gate = w = None
    eps = 0.0
    if norm is not None:
        w, gate, eps = norm
        out_n = torch.empty(T, H * 128, dtype=torch.bfloat16, device=dev)
    a = _KdaChunkedArgs(_ptr(conv_out), _ptr(g_raw), _ptr(b_raw), b_raw.stride(0), _ptr(A_log), _ptr(dt_bias),
                        float(lower_bound), _ptr(state), _ptr(out), _ptr(out_n), _ptr(gate),
                        gate.stride(0) if gate is not None else 0, _ptr(w), float(eps), H, 128,
                        _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions), _ptr(batch.state_slots), S,
                        state.shape[0], int(batch.max_q_len), T, int(write_state), _ptr(ws), ws.numel(),
                        _ptr(_status(dev)))
    _native.check(L.mb_kda_chunked(_C.byref(a), _stream()), "kda_chunked")
    _count(3 if norm is not None else 2)
    return out_n if norm is not None else out


def kda_recurrence(conv_out, g_raw, b_raw, A_log, dt_bias, lower_bound: float, state, batch, *, heads: int, dim: int,
                   write_state: bool = True, write_out: bool = True, norm=None):
    """Kimi delta attention over a ragged batch. conv_out [T, 3 H D] fp32 (q | k | v after conv + SiLU),
    g_raw [T, H D] fp32 (the decay projection), b_raw [T, >= H] fp32 (beta logits), A_log [H], dt_bias
    [H D], state [slots, H, D, D] fp32. l2-normalises q and k per head, applies the bounded gate law and
    the beta sigmoid, runs the per-channel gated delta rule. With ``norm = (w [D] fp32, gate [T, H D]
    bf16, eps)`` the sigmoid-gated output RMSNorm is applied too and the result is bf16; otherwise fp32
    [T, H D]."""
    T = conv_out.shape[0]
    H, D = heads, dim
    if conv_out.is_cuda and _native.available() and hasattr(_native.lib(), "mb_kda_recurrence"):
        if (write_out and D == 128 and getattr(batch, "max_q_len", 1) >= _KDA_CHUNK_MIN_TOKENS
                and hasattr(_native.lib(), "mb_kda_chunked")):
            y = _kda_chunked_cuda(conv_out, g_raw, b_raw, A_log, dt_bias, lower_bound, state, batch, H, write_state, norm)
            if y is not None:
                return y
        dev = conv_out.device
        out = out_n = gate = w = None
        eps = 0.0
        if norm is not None:
            w, gate, eps = norm
            out_n = torch.empty(T, H * D, dtype=torch.bfloat16, device=dev)
        else:
            out = torch.empty(T, H * D, dtype=torch.float32, device=dev)
        a = _KdaArgs(_ptr(conv_out), _ptr(g_raw), _ptr(b_raw), b_raw.stride(0), _ptr(A_log), _ptr(dt_bias),
                     float(lower_bound), _ptr(state), _ptr(out), _ptr(out_n), _ptr(gate),
                     gate.stride(0) if gate is not None else 0, _ptr(w), float(eps), H, D,
                     _ptr(batch.q_start), _ptr(batch.q_len), _ptr(batch.positions), _ptr(batch.state_slots),
                     batch.q_len.numel(), state.shape[0], int(write_state), int(write_out), _ptr(_status(dev)))
        _native.check(_native.lib().mb_kda_recurrence(_C.byref(a), _stream()), "kda_recurrence")
        _count()
        return out_n if norm is not None else out
    HD = H * D
    out = torch.zeros(T, H, D, dtype=torch.float32, device=conv_out.device)
    qs, ql, slots, pos0 = _seq_rows(batch)
    gate_all = ref.kda_gate(g_raw.view(T, H, D), A_log, dt_bias.view(H, D), lower_bound)
    beta_all = torch.sigmoid(b_raw[:, :H].float())
    for s in range(len(ql)):
        S = state[slots[s]:slots[s] + 1].clone()
        if pos0[s] == 0:
            S.zero_()
        for t in range(qs[s], qs[s] + ql[s]):
            q = ref.l2_norm(conv_out[t, :HD].view(1, H, D))
            k = ref.l2_norm(conv_out[t, HD:2 * HD].view(1, H, D))
            v = conv_out[t, 2 * HD:3 * HD].view(1, H, D)
            o, S = ref.kda_recurrence_step(S, q, k, v, gate_all[t:t + 1], beta_all[t:t + 1])
            out[t] = o[0]
        if write_state and ql[s] > 0:
            state[slots[s]] = S[0]
    if norm is not None:
        w, gate, eps = norm
        return ref.sigmoid_gated_rmsnorm(out, gate.view(T, H, D), w, eps).reshape(T, HD).to(torch.bfloat16)
    return out.reshape(T, HD)
