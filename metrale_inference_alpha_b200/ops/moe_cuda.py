"""CUDA path of the MoE ops: device routing, expert sort + tile work-list, gathered
activations, grouped tcgen05 GEMMs, weighted combine. No host synchronisation anywhere, so a
MoE layer can sit inside a CUDA graph."""
from __future__ import annotations

import ctypes as C

import torch

from . import Act, NATIVE_ACT_FOR_WEIGHT as ACT_FOR_WEIGHT, IN_RELU2, IN_SILU_MUL, _count, _native, _ptr, _stream, linear, row_op

c = C
_native.register_optional("mb_moe_route", [c.c_void_p, c.c_longlong, c.c_int, c.c_int, c.c_int, c.c_int, c.c_void_p,
                                          c.c_int, c.c_int, c.c_int, c.c_float, c.c_void_p, c.c_void_p, c.c_void_p])
_native.register_optional("mb_moe_sort", [c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int] + [c.c_void_p] * 6 +
                          [c.c_int, c.c_void_p, c.c_void_p])
_native.register_optional("mb_moe_sort_aligned", [c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int] +
                          [c.c_void_p] * 6 + [c.c_int, c.c_void_p, c.c_void_p])
_native.register_optional("mb_moe_gather_nvfp4", [c.c_void_p, c.c_longlong, c.c_void_p, c.c_longlong, c.c_int, c.c_void_p,
                                                 c.c_int, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p,
                                                 c.c_void_p, c.c_int, c.c_void_p])
_native.register_optional("mb_moe_gather", [c.c_void_p, c.c_longlong, c.c_void_p, c.c_longlong, c.c_int, c.c_void_p,
                                           c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                                           c.c_int, c.c_void_p])
_native.register_optional("mb_moe_combine", [c.c_void_p, c.c_longlong, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                                            c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p])


_native.register_optional("mb_moe_finish", [c.c_void_p, c.c_longlong, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int,
                                           c.c_void_p, c.c_longlong, c.c_void_p, c.c_longlong, c.c_void_p, c.c_void_p,
                                           c.c_void_p])


_native.register_optional("mb_moe_route_shared", [c.c_void_p, c.c_longlong, c.c_int, c.c_int, c.c_int, c.c_int, c.c_void_p,
                                                 c.c_int, c.c_int, c.c_int, c.c_float, c.c_void_p, c.c_void_p,
                                                 c.c_int, c.c_int, c.c_void_p])


def route_shared_cuda(logits: torch.Tensor, cfg, bias, shared_id: int, gate_col: int):
    """Routing over the first `num_experts` logit columns plus an always-on slot for the shared
    expert: returns weights / ids [T, k + 1]."""
    T = logits.shape[0]
    E, K = cfg.num_experts, cfg.experts_per_token
    w = torch.empty(T, K + 1, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, K + 1, dtype=torch.int32, device=logits.device)
    mode = 0 if cfg.router == "softmax" else 1
    rc = _native.lib().mb_moe_route_shared(_ptr(logits), logits.stride(0), T, E, K, mode, _ptr(bias),
                                           cfg.router_n_group if mode else 1, cfg.router_topk_group if mode else 1,
                                           int(cfg.router_renormalize), float(cfg.router_scaling if mode else 1.0),
                                           _ptr(w), _ptr(idx), shared_id, gate_col, _stream())
    _native.check(rc, "moe_route_shared")
    _count()
    return w, idx


def route_cuda(logits: torch.Tensor, cfg, bias=None):
    T, E = logits.shape
    K = cfg.experts_per_token
    w = torch.empty(T, K, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, K, dtype=torch.int32, device=logits.device)
    mode = 0 if cfg.router == "softmax" else 1
    rc = _native.lib().mb_moe_route(_ptr(logits), logits.stride(0), T, E, K, mode, _ptr(bias),
                                    cfg.router_n_group if mode else 1, cfg.router_topk_group if mode else 1,
                                    int(cfg.router_renormalize), float(cfg.router_scaling if mode else 1.0),
                                    _ptr(w), _ptr(idx), _stream())
    _native.check(rc, "moe_route")
    _count()
    return w, idx


class SortedPairs:
    """Device-side result of sorting (token, slot) pairs by local expert. With `align` > 1 every tile starts at
    a multiple of `align` rows and holds up to `tile_rows` pairs; `rows_cap` is the number of rows the sorted
    layout can then take, and every row of it that holds no pair has row_pair = -1."""

    def __init__(self, idx: torch.Tensor, expert_lo: int, num_local: int, tile_rows: int, align: int = 1):
        dev = idx.device
        T, K = idx.shape
        self.T, self.K, self.pairs = T, K, T * K
        self.tile_rows = tile_rows
        self.max_tiles = (self.pairs + tile_rows - 1) // tile_rows + num_local
        self.rows_cap = self.pairs if align == 1 else self.max_tiles * align
        i32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
        self.pair_row, self.row_pair = i32(self.pairs), i32(self.rows_cap)
        self.expert_off = i32(num_local + 1)
        self.tile_expert, self.tile_row0, self.tile_nrows = i32(self.max_tiles), i32(self.max_tiles), i32(self.max_tiles)
        self.total_rows = i32(1)
        rc = _native.lib().mb_moe_sort_aligned(_ptr(idx), self.pairs, expert_lo, num_local, tile_rows, align, self.rows_cap,
                                               _ptr(self.pair_row), _ptr(self.row_pair), _ptr(self.expert_off),
                                               _ptr(self.tile_expert), _ptr(self.tile_row0), _ptr(self.tile_nrows),
                                               self.max_tiles, _ptr(self.total_rows), _stream())
        _native.check(rc, "moe_sort")
        _count()


def gather_act(a: Act, sp: SortedPairs) -> Act:
    """Expert-sorted copy of the activation rows (and their scales)."""
    dev = a.data.device
    if a.fmt == "nvfp4":
        # one CTA per pair: packed row, per-token scale and the scale-factor words, the latter moved between the
        # 128-row tiles of the two layouts; rows without a pair are left unwritten (the GEMM stores nothing for them)
        rows = sp.rows_cap
        out = Act("nvfp4", rows, a.K, torch.empty(rows, a.data.shape[1], dtype=torch.uint8, device=dev))
        out.scale = torch.empty(rows, dtype=torch.float32, device=dev)
        out.sf_k64 = a.sf_k64
        out.sf = torch.empty((rows // 128) * a.sf_k64 * 512, dtype=torch.uint8, device=dev)
        rc = _native.lib().mb_moe_gather_nvfp4(_ptr(a.data), a.data.stride(0), _ptr(out.data), out.data.stride(0),
                                               a.data.shape[1], _ptr(sp.pair_row), sp.pairs, sp.K, rows,
                                               _ptr(a.scale), _ptr(out.scale), _ptr(a.sf), _ptr(out.sf), a.sf_k64,
                                               _stream())
        _native.check(rc, "moe_gather_nvfp4")
        _count()
        return out
    rows = sp.pairs
    alloc = rows + 64                                   # the last tile may read past the end
    row_bytes = a.data.shape[1] * a.data.element_size()
    out = Act(a.fmt, rows, a.K, torch.empty(alloc, a.data.shape[1], dtype=a.data.dtype, device=dev))
    src_scale = dst_scale = None
    groups = s_ld = d_ld = 0
    if a.fmt == "fp8_g128":
        groups, s_ld, d_ld = a.scale.shape[0], a.scale.stride(0), alloc
        # rows past the sorted pairs only feed output rows nobody reads: their scales may hold anything
        out.scale = torch.empty(groups, alloc, dtype=torch.float32, device=dev)
        src_scale, dst_scale = a.scale, out.scale
    elif a.fmt == "fp8_row":
        groups, s_ld, d_ld = 1, a.scale.numel(), alloc
        out.scale = torch.empty(alloc, dtype=torch.float32, device=dev)
        src_scale, dst_scale = a.scale, out.scale
    rc = _native.lib().mb_moe_gather(_ptr(a.data), a.data.stride(0) * a.data.element_size(), _ptr(out.data),
                                     out.data.stride(0) * out.data.element_size(), row_bytes, _ptr(sp.row_pair),
                                     sp.K, _ptr(sp.total_rows), rows, _ptr(src_scale), _ptr(dst_scale), groups,
                                     s_ld, d_ld, _stream())
    _native.check(rc, "moe_gather")
    _count()
    return out


def grouped_ffn(cfg, a: Act, weights: torch.Tensor, idx: torch.Tensor, w, finish=None) -> torch.Tensor:
    """Routed experts for all tokens: fp32 [T, hidden] = sum_j weight_j * expert_j(x). With
    `finish` = (shared bf16 [T, hidden] | None, gate logit fp32 [T, 1] | None, residual bf16 | None)
    the combine kernel also adds the (sigmoid-gated) shared expert and the residual and returns
    the bf16 block output."""
    ge = w.grouped
    T = a.M
    per_expert = max(1, (T * cfg.experts_per_token) // max(1, ge.num))
    nvfp4 = ge.gate_up.fmt == "nvfp4"
    # NVFP4: every token tile starts on a 128-row block of scale factors and takes its first tile_rows rows
    tile_rows = 16 if per_expert <= 16 else (32 if per_expert <= 32 else (64 if per_expert <= 64 or not nvfp4 else 128))
    sp = SortedPairs(idx, w.expert_lo, ge.num, tile_rows, align=128 if nvfp4 else 1)
    xa = gather_act(a, sp)
    g = lambda n: (sp.tile_expert, sp.tile_row0, sp.tile_nrows, n, sp.max_tiles, tile_rows)
    live = sp.pair_row if nvfp4 else None       # the aligned layout is mostly padding at decode sizes: one CTA per pair
    fmt_d = ACT_FOR_WEIGHT[ge.down.fmt]
    if cfg.ffn_act == "relu2":
        h = row_op(linear(xa, ge.gate_up, grouped=g(ge.n_gate_up)), fmt_d, IN_RELU2, row_index=live)[0]
    elif ge.interleaved:
        act = linear(xa, ge.gate_up, swiglu=True, grouped=g(ge.n_gate_up))
        h = row_op(act, fmt_d, scale_pad=64, row_index=live)[0]
    else:
        h = row_op(linear(xa, ge.gate_up, grouped=g(ge.n_gate_up)), fmt_d, IN_SILU_MUL, scale_pad=64, row_index=live)[0]
    if cfg.ffn_act == "relu2" and h.fmt == "fp8_g128" and h.scale.shape[1] < h.M + 64:
        pad = torch.empty(h.scale.shape[0], h.M + 64, dtype=torch.float32, device=h.scale.device)
        pad[:, :h.scale.shape[1]] = h.scale
        h.scale = pad
    y = linear(h, ge.down, out_f32=True, grouped=g(ge.n_down))
    if finish is not None:
        shared, gate, residual = finish
        out = torch.empty(T, ge.n_down, dtype=torch.bfloat16, device=y.device)
        rc = _native.lib().mb_moe_finish(_ptr(y), y.stride(0), _ptr(sp.pair_row), _ptr(weights), T, sp.K, ge.n_down,
                                         _ptr(shared), shared.stride(0) if shared is not None else 0,
                                         _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(residual),
                                         _ptr(out), _stream())
        _native.check(rc, "moe_finish")
        _count()
        return out
    out = torch.empty(T, ge.n_down, dtype=torch.float32, device=y.device)
    rc = _native.lib().mb_moe_combine(_ptr(y), y.stride(0), _ptr(sp.pair_row), _ptr(weights), T, sp.K, ge.n_down,
                                      None, _ptr(out), None, _stream())
    _native.check(rc, "moe_combine")
    _count()
    return out
