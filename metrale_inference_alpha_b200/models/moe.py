"""MoE FFN block: norm -> router -> top-k -> routed experts (+ shared expert, optional
sigmoid gate) -> blend -> residual (``kernels/circuits/qwen3_6_moe.toml:43-125``; sigmoid
group-limited routing for DeepSeek-V3-shaped models).

Expert parallelism: every rank routes all tokens; on the plain path a rank runs only its
local experts and the partial outputs are summed over ranks (the reference's masked-local +
all-reduce scheme, ``model-layers/src/layers/moe/forward/ep_reduce.rs:21-52``). The fused
dispatch/combine path over NVLink peer memory lives in ``parallel/ep.py``.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import NATIVE_ACT_FOR_WEIGHT as ACT_FOR_WEIGHT, moe as moe_ops   # experts keep the weight's own activation format


def moe_block(dec, x, lw):
    c, w = dec.cfg, lw.ffn
    if getattr(w, "paged", None) is not None:
        fmt = ACT_FOR_WEIGHT[w.paged.spec.fmt[0]]
    else:
        fmt = ACT_FOR_WEIGHT[(w.experts[0].gate_up if w.experts else w.shared.gate_up).fmt]
    a = dec._norm_act(x, lw.ln2, fmt, also_bf16=True, res_only=dec.tp.size > 1)
    x = dec.res(x)
    hb = a.bf16
    T = x.shape[0]
    ep = getattr(dec.tp, "ep", None)
    ge = w.grouped
    if x.is_cuda and ep is None and ge is not None and ge.shared_slot is not None:
        # the shared expert is stacked behind the routed ones and the router weight carries its gate
        # row: one routing launch hands every token k + 1 (expert, weight) pairs, and the grouped
        # GEMMs, the sort and the combine serve the shared expert at no extra launch
        from ..ops.moe_cuda import grouped_ffn, route_shared_cuda
        logits = ops.linear(dec._as_act(hb, "bf16"), w.router_ext, out_f32=True)
        weights, idx = route_shared_cuda(logits, c, w.bias, w.expert_lo + ge.shared_slot,
                                         c.num_experts if w.shared_gate is not None else -1)
        if dec.tp.size > 1:
            return dec.tp.sum_deferred(grouped_ffn(c, a, weights, idx, w, finish=(None, None, None)), residual=x)
        return grouped_ffn(c, a, weights, idx, w, finish=(None, None, x))
    logits = ops.linear(dec._as_act(hb, "bf16"), w.router, out_f32=True)
    weights, idx = moe_ops.route(logits, c, w.bias)
    replicated = w.shared is not None and getattr(w, "shared_replicated", False) and dec.tp.size > 1
    if (x.is_cuda and ep is None and w.grouped is not None and not replicated
            and (w.shared is None or w.shared_gate is None or w.shared_gate.N == 1)):
        # CUDA fast path: the combine kernel also applies the shared expert's sigmoid gate and adds
        # the residual, so the block's tail is one launch instead of a chain of elementwise ops
        from ..ops.moe_cuda import grouped_ffn
        sh = shared_expert(dec, a, w) if w.shared is not None else None
        g = ops.linear(dec._as_act(hb, "bf16"), w.shared_gate, out_f32=True) if (sh is not None and w.shared_gate is not None) else None
        if dec.tp.size > 1:
            y = grouped_ffn(c, a, weights, idx, w, finish=(sh, g, None))
            return dec.tp.sum_deferred(y, residual=x)
        return grouped_ffn(c, a, weights, idx, w, finish=(sh, g, x))
    if ep is not None and x.is_cuda:
        routed = ep.dispatch_compute_combine(dec, a, weights, idx, w)
    else:
        routed = routed_experts(dec, a, weights, idx, w)
    y = routed
    sh = None
    if w.shared is not None:
        sh = shared_expert(dec, a, w)
        if w.shared_gate is not None:
            g = ops.linear(dec._as_act(hb, "bf16"), w.shared_gate, out_f32=True)
            sh = sh.float() * torch.sigmoid(g)
    # a width-sharded shared expert is a partial sum like the routed part; a replicated one (expert
    # parallelism) is added once, after the sum over ranks
    if sh is not None and not replicated:
        y = y.float() + sh.float()
    if dec.tp.size > 1:
        # the sum over ranks (+ residual) is left to the next norm when the fused reduction is on
        res = (x.float() + sh.float()).to(torch.bfloat16) if replicated else x
        return dec.tp.sum_deferred(y.to(torch.bfloat16), residual=res)
    return (x.float() + y.float()).to(torch.bfloat16)


def shared_expert(dec, a, w):
    f = w.shared
    fmt_d = ACT_FOR_WEIGHT[f.down.fmt]
    if dec.cfg.ffn_act == "relu2":
        h = ops.row_op(ops.linear(a, f.gate_up), fmt_d, ops.IN_RELU2)[0]
    elif f.interleaved:
        h = dec._as_act(ops.linear(a, f.gate_up, swiglu=True), fmt_d)
    else:
        h = ops.row_op(ops.linear(a, f.gate_up), fmt_d, ops.IN_SILU_MUL)[0]
    return ops.linear(h, f.down)


def routed_experts(dec, a, weights, idx, w):
    """Sum over the local experts of weight * expert(x); fp32 [T, hidden]."""
    if getattr(w, "paged", None) is not None:
        return _routed_paged(dec, a, weights, idx, w)
    if a.data.is_cuda and w.grouped is not None:
        from ..ops.moe_cuda import grouped_ffn
        return grouped_ffn(dec.cfg, a, weights, idx, w)
    T = a.M
    H = dec.cfg.hidden_size
    out = torch.zeros(T, H, dtype=torch.float32, device=a.data.device)
    lo = w.expert_lo
    for j, f in enumerate(w.experts):
        e = lo + j
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        if a.data.is_cuda and a.fmt != "bf16":
            # a quantised activation keeps its scales in a layout tied to the row order: the expert's rows
            # are re-encoded from the bf16 copy
            sub = dec._as_act(a.bf16[tok].contiguous(), ACT_FOR_WEIGHT[f.gate_up.fmt])
        else:
            sub = ops.Act(a.fmt, tok.numel(), a.K, a.data[tok])
        fmt_d = ACT_FOR_WEIGHT[f.down.fmt]
        if dec.cfg.ffn_act == "relu2":
            h = ops.row_op(ops.linear(sub, f.gate_up), fmt_d, ops.IN_RELU2)[0]
        elif f.interleaved:
            h = ops.quantize_act(ops.linear(sub, f.gate_up, swiglu=True), fmt_d)
        else:
            h = ops.row_op(ops.linear(sub, f.gate_up), fmt_d, ops.IN_SILU_MUL)[0]
        y = ops.linear(h, f.down, out_f32=True)
        out.index_add_(0, tok, y * weights[tok, slot][:, None])
    return out


def _routed_paged(dec, a, weights, idx, w):
    """Routed experts whose weights are paged from an expert store: every wave of resident experts is
    one pass of the grouped (CUDA) or per-expert (CPU) path over the routing ids rewritten to arena
    slots; experts outside the wave carry id -1 and are dropped, and the waves' outputs add up."""
    import copy
    paged = w.paged
    out = None
    for slot_idx in paged.waves(w.paged_layer, idx):
        view = copy.copy(w)
        view.paged, view.expert_lo = None, 0
        if a.data.is_cuda:
            view.grouped, view.experts = paged.grouped, []
        else:
            view.grouped = None
            view.experts = [paged.slot_ffn(s) if paged.resident[s] is not None else None for s in range(paged.slots)]
        y = _routed_slots(dec, a, weights, slot_idx, view)
        out = y if out is None else out + y
    if out is None:
        out = torch.zeros(a.M, dec.cfg.hidden_size, dtype=torch.float32, device=a.data.device)
    return out


def _routed_slots(dec, a, weights, idx, view):
    if view.grouped is not None:
        from ..ops.moe_cuda import grouped_ffn
        return grouped_ffn(dec.cfg, a, weights, idx, view)
    live = [(j, f) for j, f in enumerate(view.experts) if f is not None]
    T, H = a.M, dec.cfg.hidden_size
    out = torch.zeros(T, H, dtype=torch.float32, device=a.data.device)
    for j, f in live:
        tok, slot = torch.nonzero(idx == j, as_tuple=True)
        if tok.numel() == 0:
            continue
        sub = ops.Act(a.fmt, tok.numel(), a.K, a.data[tok])
        fmt_d = ACT_FOR_WEIGHT[f.down.fmt]
        if dec.cfg.ffn_act == "relu2":
            h = ops.row_op(ops.linear(sub, f.gate_up), fmt_d, ops.IN_RELU2)[0]
        elif f.interleaved:
            h = ops.quantize_act(ops.linear(sub, f.gate_up, swiglu=True), fmt_d)
        else:
            h = ops.row_op(ops.linear(sub, f.gate_up), fmt_d, ops.IN_SILU_MUL)[0]
        y = ops.linear(h, f.down, out_f32=True)
        out.index_add_(0, tok, y * weights[tok, slot][:, None])
    return out
