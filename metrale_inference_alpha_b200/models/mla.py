"""Multi-head latent attention block (DeepSeek-V3 shape) in absorbed form.

The paged cache stores one row per token: ``[kv_lora latent (RMS-normed) | rope key]``
(kv_lora + rope dims, a single "kv head"). Queries are projected into latent space with
W_uk, attention runs as multi-query attention over the latent rows, and W_uv maps the
latent-space output back to per-head values before o_proj.
On a GPU the block is: projections (tcgen05 GEMMs), the two absorption products as bf16 batched
GEMMs over heads, one assembly kernel (latent RMSNorm, both rotations, cache row write, absorbed
query rows: ``mla.cu::mla_prepare_kernel``) and the paged attention kernel (one CTA per 16 query
rows, the cached tile feeding both products); this file keeps the fp32 restatement used on CPU
and as the oracle.
Reference behaviour: ``kernels/gb10/deepseek-v4-flash/nvfp4/mla_absorbed.cu``
(``mla_batched_gemv``, ``mla_cache_assemble``), ``paged_decode_attn_mla.cu``.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..ops import ACT_FOR_WEIGHT, mla_cuda, sparse_attn
from ..ops import reference as ref


def mla_block(dec, x, lw, batch, kv, j: int):
    c, w = dec.cfg, lw.mixer
    H, nope, rope, vd, L = w.heads, c.qk_nope_dim, c.qk_rope_dim, c.v_head_dim, c.kv_lora_rank
    T = x.shape[0]
    a = dec._norm_act(x, lw.ln1, ACT_FOR_WEIGHT[w.kv_a.fmt], also_bf16=w.idx_q is not None, res_only=True)
    x = dec.res(x)
    sel = None
    if w.q_a is not None:
        qa = ops.linear(a, w.q_a)
        want_lat = w.idx_q is not None
        qn = ops.row_op(qa, ACT_FOR_WEIGHT[w.q_b.fmt], ops.IN_RMSNORM, w=w.q_a_norm, eps=c.rms_eps,
                        **({"also_bf16": True} if want_lat and ACT_FOR_WEIGHT[w.q_b.fmt] != "bf16" else {}))[0]
        q = ops.linear(qn, w.q_b)
    else:
        qn = None
        q = ops.linear(a, w.q_b)
    if w.idx_q is not None:
        sel = _index_select(dec, x, a, qn, w, batch, kv, j)
    scale = 1.0 / math.sqrt(nope + rope)
    sc = c.rope_scaling or {}
    if sc.get("rope_type", sc.get("type")) == "yarn" and sc.get("mscale_all_dim"):
        # DeepSeek long-context checkpoints fold the YaRN magnitude correction into the softmax scale
        m = 0.1 * float(sc["mscale_all_dim"]) * math.log(float(sc.get("factor", 1.0))) + 1.0
        scale *= m * m
    if (x.is_cuda and L == mla_cuda.LATENT and kv.k[j].dtype == torch.bfloat16 and kv.k[j].shape[-1] == mla_cuda.ROW
            and dec.cos.shape[1] * 2 == rope and w.kv_a_norm.dtype == torch.bfloat16):
        # GPU: bf16 absorption products on the tensor cores (batched over heads), one kernel for the
        # latent norm + both rotations + the cache write + the query assembly, the paged MLA kernel
        q = q.view(T, H, nope + rope)
        ckv = ops.linear(a, w.kv_a)                                    # [T, L + rope] bf16
        uk = _bf16(w, "w_uk")                                          # [H, nope, L]
        q_lat = torch.bmm(q[..., :nope].transpose(0, 1), uk)           # [H, T, L]
        qq = mla_cuda.prepare(q, q_lat, ckv, w.kv_a_norm, dec.cos, dec.sin, batch.positions, batch.slot_mapping,
                              kv.k[j], nope, c.rms_eps)
        if sel is not None:
            o_lat = sparse_attn.selected_latent_attention(qq, kv.k[j], batch.block_table, sel[0], sel[1], sel[2], scale, L)
        else:
            o_lat = mla_cuda.mla_attention(qq, kv.k[j], batch.block_table, batch.q_start, batch.q_len, batch.ctx_len,
                                           max_q_len=batch.max_q_len, max_ctx=max(batch.max_ctx, 1), scale=scale)
        uv = _bf16(w, "w_uv")                                          # [H, vd, L]
        o = torch.bmm(o_lat.to(torch.bfloat16).transpose(0, 1), uv.transpose(1, 2))      # [H, T, vd]
        o = o.transpose(0, 1).reshape(T, H * vd)
        oa = ops.quantize_act(o, ACT_FOR_WEIGHT[w.o.fmt])
        return dec.tp.linear_reduce(oa, w.o, residual=x, defer=True)
    q = q.view(T, H, nope + rope).float()
    ckv = ops.linear(a, w.kv_a).float()                                # [T, L + rope]
    lat = ref.rms_norm(ckv[:, :L], w.kv_a_norm, c.rms_eps)
    k_rope = ref.apply_rope_neox(ckv[:, None, L:], batch.positions, dec.cos, dec.sin)[:, 0]
    q_rope = ref.apply_rope_neox(q[..., nope:], batch.positions, dec.cos, dec.sin)
    row = torch.cat([lat, k_rope], -1).to(kv.k[j].dtype)               # cache row
    flat = kv.k[j].view(-1, L + rope)
    # rows without a slot (-1: padding of a CUDA-graph rung) land in the reserved null block 0, which
    # no sequence reads; a fixed-shape scatter keeps the step capturable
    flat.index_copy_(0, batch.slot_mapping.clamp(min=0), row)
    q_lat = torch.einsum("thn,hnl->thl", q[..., :nope], w.w_uk.float())   # absorb W_uk
    qq = torch.cat([q_lat, q_rope], -1).to(torch.bfloat16)             # [T, H, L + rope]
    if sel is not None:
        o_lat = sparse_attn.selected_latent_attention(qq, kv.k[j], batch.block_table, sel[0], sel[1], sel[2], scale, L)
    elif mla_cuda.supported(qq, kv.k[j]) and L == mla_cuda.LATENT:
        o_lat = mla_cuda.mla_attention(qq, kv.k[j], batch.block_table, batch.q_start, batch.q_len, batch.ctx_len,
                                       max_q_len=batch.max_q_len, max_ctx=max(batch.max_ctx, 1), scale=scale)
    else:
        o_lat = mla_attention(qq, kv.k[j], batch, scale, L)            # [T, H, L] fp32
    o = torch.einsum("thl,hvl->thv", o_lat, w.w_uv.float()).reshape(T, H * vd)
    oa = ops.quantize_act(o.to(torch.bfloat16), ACT_FOR_WEIGHT[w.o.fmt])
    return dec.tp.linear_reduce(oa, w.o, residual=x, defer=True)


def _index_select(dec, x, a, qn, w, batch, kv, j: int):
    """The sparse-attention indexer of one layer: writes this step's indexer keys into the pool's second
    tensor and, when some row sees more than ``index_topk`` tokens, returns (row -> sequence, selected
    positions [T, k], count [T]); None means every row attends to its whole context (dense attention is
    then exactly what the selection would give). Indexer queries come from the query latent, keys and
    head weights from the block input; q / k are rotated on their first ``qk_rope_dim`` dims; the key goes
    through a LayerNorm. score = sum_h w_h relu(q_h . k), with w scaled by Hi^-1/2 Di^-1/2."""
    c = dec.cfg
    Hi, Di = c.index_n_heads, c.index_head_dim
    T = x.shape[0]
    hb = _plain(a)
    src = hb if qn is None else _plain(qn)
    iq = ops.linear(dec._as_act(src, "bf16"), w.idx_q, out_f32=True).view(T, Hi, Di)
    ik = ops.linear(dec._as_act(hb, "bf16"), w.idx_k, out_f32=True)                       # [T, Di]
    ik = torch.nn.functional.layer_norm(ik, (Di,), w.idx_k_norm[0], w.idx_k_norm[1], 1e-6)
    iw = ops.linear(dec._as_act(hb, "bf16"), w.idx_w, out_f32=True) * (Hi ** -0.5 * Di ** -0.5)
    iq = ref.apply_rope_neox(iq, batch.positions, dec.cos, dec.sin)          # the first qk_rope_dim channels rotate
    ik = ref.apply_rope_neox(ik[:, None], batch.positions, dec.cos, dec.sin)[:, 0]
    kc = kv.v[j]
    kc.view(-1, Di).index_copy_(0, batch.slot_mapping.clamp(min=0), ik.to(kc.dtype))
    if batch.max_ctx <= c.index_topk:
        return None
    row_seq, row_ctx = sparse_attn.row_meta(batch)
    scores = sparse_attn.index_scores(iq.to(torch.bfloat16), iw.float(), kc, batch.block_table, row_seq, row_ctx,
                                      batch.max_ctx)
    idx, cnt = sparse_attn.topk_indices(scores, row_ctx, c.index_topk)
    return row_seq, idx, cnt


def _plain(act) -> torch.Tensor:
    """The unquantised values of an activation: its bf16 side copy, or its data when that is already
    plain (bf16 activations; every activation on the CPU path)."""
    if getattr(act, "bf16", None) is not None:
        return act.bf16
    if act.fmt == "bf16" or not act.data.is_cuda:
        return act.data
    raise ValueError("the indexer needs the unquantised activation (request also_bf16)")


def _bf16(w, name: str) -> torch.Tensor:
    """The absorption matrix as a bf16 tensor, converted once and kept beside the weights."""
    key = "_" + name + "_bf16"
    t = getattr(w, key, None)
    if t is None:
        t = getattr(w, name).to(torch.bfloat16).contiguous()
        setattr(w, key, t)
    return t


def mla_attention(q, cache, batch, scale: float, L: int) -> torch.Tensor:
    """Multi-query attention over latent rows: keys are the full row, values its first L dims."""
    T, H, D = q.shape
    nb, bs, _, _ = cache.shape
    out = torch.zeros(T, H, L, dtype=torch.float32, device=q.device)
    qs, ql, cl = batch.q_start.tolist(), batch.q_len.tolist(), batch.ctx_len.tolist()
    for s in range(len(ql)):
        n, ctx = ql[s], cl[s]
        if n <= 0:
            continue
        nblk = (ctx + bs - 1) // bs
        rows = cache[batch.block_table[s, :nblk].long()].reshape(nblk * bs, D)[:ctx].float()
        qq = q[qs[s]:qs[s] + n].float()
        sc = torch.einsum("qhd,kd->hqk", qq, rows) * scale
        pq = torch.arange(ctx - n, ctx, device=q.device)[:, None]
        pk = torch.arange(ctx, device=q.device)[None, :]
        sc = sc.masked_fill(~(pk <= pq)[None], float("-inf"))
        out[qs[s]:qs[s] + n] = torch.einsum("hqk,kl->qhl", torch.softmax(sc, -1), rows[:, :L])
    return out
