"""Loaders for the non-dense modules: gated-delta-net, Mamba2, MoE, MLA, Nemotron-H stack."""
from __future__ import annotations

import torch

from .. import ops
from ..ops import QuantWeight
from .loader import (FfnW, GdnW, LayerW, MambaW, MlaW, ModelW, MoeW, finalize, slice_cols, slice_rows)


def _ep_range(ld):
    E = ld.cfg.num_experts
    per = E // ld.ep_size
    return ld.ep_rank * per, (ld.ep_rank + 1) * per


def gdn(ld, p: str) -> GdnW:
    """in_proj_qkv rows are [Q | K | V] (heads contiguous), in_proj_z rows [Z]; fused to one
    [Q | K | V | Z] GEMM; in_proj_b / in_proj_a fused to a bf16 [b | a] GEMM. Under tensor
    parallelism every segment is split by head (crates/model-arch/src/tp_shard/gdn.rs)."""
    c = ld.cfg
    qkv, z = ld.lin(f"{p}.in_proj_qkv"), ld.lin(f"{p}.in_proj_z")
    b, a = ld.lin(f"{p}.in_proj_b", quant=False), ld.lin(f"{p}.in_proj_a", quant=False)
    out = ld.lin(f"{p}.out_proj")
    conv = ld.src.get(f"{p}.conv1d.weight").to(ld.dev).float().reshape(-1, c.conv_kernel)
    QK, V = c.gdn_qk_size, c.gdn_v_size
    kh, vh = c.gdn_k_heads, c.gdn_v_heads
    A_log, dt_bias = ld.vec(f"{p}.A_log", torch.float32), ld.vec(f"{p}.dt_bias", torch.float32)
    if ld.tp_size > 1:
        klo, khi = ld._shard(kh)
        vlo, vhi = ld._shard(vh)
        kd, vd = c.gdn_k_dim, c.gdn_v_dim
        segs = [(klo * kd, khi * kd), (QK + klo * kd, QK + khi * kd), (2 * QK + vlo * vd, 2 * QK + vhi * vd)]
        qkv = ops.concat_weights([slice_rows(qkv, lo, hi) for lo, hi in segs])
        conv = torch.cat([conv[lo:hi] for lo, hi in segs], 0)
        z = slice_rows(z, vlo * vd, vhi * vd)
        b, a = slice_rows(b, vlo, vhi), slice_rows(a, vlo, vhi)
        out = slice_cols(out, vlo * vd, vhi * vd)
        A_log, dt_bias = A_log[vlo:vhi].contiguous(), dt_bias[vlo:vhi].contiguous()
        kh, vh = khi - klo, vhi - vlo
    return GdnW(finalize(ops.concat_weights([qkv, z])), ops.concat_weights([b, a]), conv.contiguous(),
                A_log, dt_bias, ld.vec(f"{p}.norm.weight"), finalize(out), kh, vh)


def kda(ld, p: str):
    """Kimi delta attention block: q / k / v projections fused to one GEMM, their three short
    convolutions concatenated in the same q | k | v order, the low-rank decay (f_a, f_b) and output-gate
    (g_a, g_b) projections, per-channel dt_bias and per-head A_log in fp32. Tensor parallelism splits
    every per-head tensor by head and leaves the rank-sized inner projections replicated
    (crates/model-arch/src/glm5next_kda/{binding,tp}.rs)."""
    from .loader import KdaW
    c = ld.cfg
    H, D = c.kda_heads, c.kda_head_dim
    q, k, v = (ld.lin(f"{p}.{n}_proj") for n in "qkv")
    conv = [ld.src.get(f"{p}.{n}_conv1d.weight").to(ld.dev).float().reshape(-1, c.conv_kernel) for n in "qkv"]
    f_a, f_b = ld.lin(f"{p}.f_a_proj", quant=False), ld.lin(f"{p}.f_b_proj", quant=False)
    g_a, g_b = ld.lin(f"{p}.g_a_proj", quant=False), ld.lin(f"{p}.g_b_proj", quant=False)
    b = ld.lin(f"{p}.b_proj", quant=False)
    out = ld.lin(f"{p}.o_proj")
    A_log = ld.vec(f"{p}.A_log", torch.float32).reshape(-1)
    dt_bias = ld.vec(f"{p}.dt_bias", torch.float32).reshape(-1)
    if ld.tp_size > 1:
        lo, hi = ld._shard(H)
        rows = (lo * D, hi * D)
        q, k, v = (slice_rows(w, *rows) for w in (q, k, v))
        conv = [cw[rows[0]:rows[1]] for cw in conv]
        f_b, g_b = slice_rows(f_b, *rows), slice_rows(g_b, *rows)
        b = slice_rows(b, lo, hi)
        out = slice_cols(out, *rows)
        A_log, dt_bias = A_log[lo:hi].contiguous(), dt_bias[rows[0]:rows[1]].contiguous()
        H = hi - lo
    return KdaW(finalize(ops.concat_weights([q, k, v])), f_a, f_b, b, g_a, g_b, torch.cat(conv, 0).contiguous(),
                A_log, dt_bias, ld.vec(f"{p}.o_norm.weight", torch.float32), finalize(out), H)


def mamba2(ld, p: str) -> MambaW:
    """in_proj rows are [z | x | B | C | dt]; tensor parallelism splits heads (z, x, dt) and
    state groups (B, C) together."""
    c = ld.cfg
    inp, out = ld.lin(f"{p}.in_proj"), ld.lin(f"{p}.out_proj")
    conv = ld.src.get(f"{p}.conv1d.weight").to(ld.dev).float().reshape(-1, c.conv_kernel)
    conv_b = ld.vec(f"{p}.conv1d.bias", torch.float32) if ld.src.has(f"{p}.conv1d.bias") else None
    A_log, D, dtb = (ld.vec(f"{p}.{n}", torch.float32) for n in ("A_log", "D", "dt_bias"))
    norm_w = ld.vec(f"{p}.norm.weight")
    H, G, inner, GN = c.mamba_heads, c.mamba_groups, c.mamba_inner, c.mamba_groups * c.mamba_state
    if ld.tp_size > 1:
        hlo, hhi = ld._shard(H)
        glo, ghi = ld._shard(G)
        P, N = c.mamba_head_dim, c.mamba_state
        xs = (hlo * P, hhi * P)
        segs = [(xs[0], xs[1]), (inner + xs[0], inner + xs[1]),
                (2 * inner + glo * N, 2 * inner + ghi * N), (2 * inner + GN + glo * N, 2 * inner + GN + ghi * N),
                (2 * inner + 2 * GN + hlo, 2 * inner + 2 * GN + hhi)]
        inp = ops.concat_weights([slice_rows(inp, lo, hi) for lo, hi in segs])
        csegs = [(xs[0], xs[1]), (inner + glo * N, inner + ghi * N), (inner + GN + glo * N, inner + GN + ghi * N)]
        conv = torch.cat([conv[lo:hi] for lo, hi in csegs], 0)
        if conv_b is not None:
            conv_b = torch.cat([conv_b[lo:hi] for lo, hi in csegs], 0)
        out = slice_cols(out, xs[0], xs[1])
        A_log, D, dtb = A_log[hlo:hhi].contiguous(), D[hlo:hhi].contiguous(), dtb[hlo:hhi].contiguous()
        norm_w = norm_w[xs[0]:xs[1]].contiguous()
        H, G = hhi - hlo, ghi - glo
    return MambaW(finalize(inp), conv.contiguous(), conv_b, A_log, D, dtb, norm_w, finalize(out), H, G)


def moe(ld, p: str) -> MoeW:
    """Router (bf16, replicated) + routed experts + shared expert. Expert parallelism keeps
    experts [lo, hi) on this rank; tensor parallelism (when ep_size == 1) splits every
    expert's FFN width instead."""
    c = ld.cfg
    w = MoeW()
    w.router = ld.lin(f"{p}.gate", quant=False)
    if ld.src.has(f"{p}.gate.e_score_correction_bias"):
        w.bias = ld.vec(f"{p}.gate.e_score_correction_bias", torch.float32)
    lo, hi = _ep_range(ld)
    w.expert_lo = lo
    shard_width = ld.ep_size == 1
    for e in range(lo, hi):
        w.experts.append(ld.ffn(f"{p}.experts.{e}", shard=shard_width))
    if c.num_shared_experts:
        sp = "shared_expert" if ld.src.has(f"{p}.shared_expert.up_proj.weight") or \
            ld.src.has(f"{p}.shared_expert.up_proj.weight_packed") else "shared_experts"
        w.shared = ld.ffn(f"{p}.{sp}", shard=shard_width)
        w.shared_replicated = not shard_width
        if ld.src.has(f"{p}.shared_expert_gate.weight"):
            w.shared_gate = ld.lin(f"{p}.shared_expert_gate", quant=False)
    if ld.dev.type == "cuda":
        from ..ops import concat_weights, moe as moe_ops
        sh = w.shared
        import os
        fold = (os.environ.get("METRALE_MOE_FOLD_SHARED", "1") != "0"
                and sh is not None and w.experts and not w.shared_replicated and lo == 0 and hi == c.num_experts
                and c.num_experts < 512 and c.experts_per_token < 31
                and sh.gate_up.N == w.experts[0].gate_up.N and sh.down.K == w.experts[0].down.K
                and sh.gate_up.fmt == w.experts[0].gate_up.fmt and sh.interleaved == w.experts[0].interleaved
                and (w.shared_gate is None or w.shared_gate.N == 1))
        w.grouped = moe_ops.stack_experts(w.experts + ([sh] if fold else []))
        if fold and w.grouped is not None:
            # the shared expert becomes expert `num_experts` of the stack (every token routes to it),
            # and its sigmoid gate row is appended to the router weight
            w.grouped.shared_slot = len(w.experts)
            parts = [w.router] + ([w.shared_gate] if w.shared_gate is not None else [])
            n = sum(p_.N for p_ in parts)
            if n % 8:                                       # logit rows stay 32-byte aligned
                from ..ops import QuantWeight
                z = torch.zeros(8 - n % 8, w.router.K, dtype=w.router.data.dtype, device=w.router.data.device)
                parts.append(QuantWeight("bf16", z.shape[0], w.router.K, z))
            w.router_ext = concat_weights(parts)
    return w


def mla(ld, p: str) -> MlaW:
    """Multi-head latent attention in absorbed form: kv_b_proj is split into W_uk
    [H, nope, kv_lora] (folded into the query) and W_uv [H, v, kv_lora] (applied to the
    latent-space attention output); both are kept in bf16."""
    c = ld.cfg
    w = MlaW()
    if ld.src.has(f"{p}.q_a_proj.weight"):
        w.q_a = finalize(ld.lin(f"{p}.q_a_proj"))
        w.q_a_norm = ld.vec(f"{p}.q_a_layernorm.weight")
        q_b = ld.lin(f"{p}.q_b_proj")
    else:
        q_b = ld.lin(f"{p}.q_proj")
    w.kv_a = finalize(ld.lin(f"{p}.kv_a_proj_with_mqa"))
    w.kv_a_norm = ld.vec(f"{p}.kv_a_layernorm.weight")
    kv_b = ld.lin(f"{p}.kv_b_proj").dequant().view(c.num_heads, c.qk_nope_dim + c.v_head_dim, c.kv_lora_rank)
    o = ld.lin(f"{p}.o_proj")
    H = c.num_heads
    qh = c.qk_nope_dim + c.qk_rope_dim
    if ld.tp_size > 1:
        lo, hi = ld._shard(H)
        q_b = slice_rows(q_b, lo * qh, hi * qh)
        kv_b = kv_b[lo:hi]
        o = slice_cols(o, lo * c.v_head_dim, hi * c.v_head_dim)
        H = hi - lo
    w.q_b, w.o, w.heads = finalize(q_b), finalize(o), H
    w.w_uk = kv_b[:, :c.qk_nope_dim].to(torch.bfloat16).contiguous()
    w.w_uv = kv_b[:, c.qk_nope_dim:].to(torch.bfloat16).contiguous()
    if c.index_topk > 0:
        q = f"{p}.indexer"
        w.idx_q = ld.lin(f"{q}.wq_b", quant=False)
        w.idx_k = ld.lin(f"{q}.wk", quant=False)
        w.idx_w = ld.lin(f"{q}.weights_proj", quant=False)
        w.idx_k_norm = torch.stack([ld.vec(f"{q}.k_norm.weight", torch.float32), ld.vec(f"{q}.k_norm.bias", torch.float32)])
    return w


def load_nemotron(ld) -> ModelW:
    c = ld.cfg
    m = ModelW()
    m.embed = ld.vec("backbone.embeddings.weight")
    m.final_norm = ld.vec("backbone.norm_f.weight")
    head = ld.lin("lm_head", quant=False)
    m.vocab_lo, m.vocab_hi = 0, c.vocab_size
    if ld.tp_size > 1:
        per = (c.vocab_size + ld.tp_size - 1) // ld.tp_size
        m.vocab_lo, m.vocab_hi = ld.tp_rank * per, min(c.vocab_size, (ld.tp_rank + 1) * per)
        head = slice_rows(head, m.vocab_lo, m.vocab_hi)
    m.lm_head = head
    b = 0
    for i in range(c.num_layers):
        L = LayerW(kind=c.layer_types[i], ffn_kind=c.ffn_types[i])
        p = f"backbone.layers.{b}"
        b += 1
        L.ln1 = ld.vec(f"{p}.norm.weight")
        if L.kind == "mamba2":
            L.mixer = mamba2(ld, f"{p}.mixer")
        else:
            # the attention loader expects {q,k,v,o}_proj under one prefix
            L.mixer = ld.attention(f"{p}.mixer")
        if L.ffn_kind != "none":
            q = f"backbone.layers.{b}"
            b += 1
            L.ln2 = ld.vec(f"{q}.norm.weight")
            L.ffn = ld.ffn(f"{q}.mixer")
        m.layers.append(L)
    return m
