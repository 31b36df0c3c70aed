"""Recurrent mixers: gated-delta-net (Qwen3.5 / 3.6 linear attention) and Mamba2 (Nemotron-H).

Both keep an fp32 state per sequence in the state pool (a conv window + a matrix) and
process a batch whose sequences contribute any number of tokens (decode 1, verify k+1,
prefill chunk n). On CUDA the conv, gate, recurrence and scan steps are the kernels in
``ops/csrc/recurrent.cu`` (one launch for all sequences); on CPU they are the reference loops.
Op order: ``kernels/circuits/blocks/qwen3_hybrid.toml:52-130`` and
``kernels/circuits/nemotron_h.toml:81-173``.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import ACT_FOR_WEIGHT
from ..ops import recurrent as rops


def gdn_block(dec, x, lw, batch, pool, sidx: int):
    c, w = dec.cfg, lw.mixer
    kd, vd, kh, vh = c.gdn_k_dim, c.gdn_v_dim, w.k_heads, w.v_heads
    QK, V = kh * kd, vh * vd
    a = dec._norm_act(x, lw.ln1, ACT_FOR_WEIGHT[w.in_qkvz.fmt], also_bf16=True, res_only=True)
    x = dec.res(x)
    qkvz = ops.linear(a, w.in_qkvz)                                   # [T, 2QK + 2V]
    ba = ops.linear(dec._as_act(a.bf16, "bf16"), w.in_ba, out_f32=True)   # [T, 2 vh] = b | a
    stash = getattr(batch, "spec_stash", None)
    ws = stash is None                                               # verify steps commit the state afterwards
    conv_out = rops.causal_conv1d(qkvz, 2 * QK + V, w.conv_w, None, pool.conv[sidx], batch, activation=True,
                                  write_state=ws)
    core = rops.gdn_recurrence(conv_out, ba, w.A_log, w.dt_bias, pool.ssm[sidx], batch,
                               k_heads=kh, v_heads=vh, k_dim=kd, v_dim=vd, write_state=ws)   # [T, V] fp32
    if stash is not None:
        stash.layers[sidx] = ("gdn", lw, qkvz, conv_out, ba)
    z = qkvz[:, 2 * QK + V:]
    y = ops.row_op(core, ACT_FOR_WEIGHT[w.out.fmt], ops.IN_GATED_RMSNORM, gate=z, w=_tile(w, w.norm_w, vh),
                   group=vd, eps=c.rms_eps)[0]
    return dec.tp.linear_reduce(y, w.out, residual=x, defer=True)


def kda_block(dec, x, lw, batch, pool, sidx: int):
    """Kimi delta attention: q|k|v projection -> short convolution + SiLU -> (inside the recurrence
    kernel) l2 norm of q and k, bounded per-channel decay from the low-rank f projection, beta =
    sigmoid(b), per-channel gated delta rule, sigmoid-gated output RMSNorm with the low-rank g
    projection -> output projection. Reference op graph: crates/model-arch/src/glm5next_kda/mod.rs."""
    c, w = dec.cfg, lw.mixer
    H, D = w.heads, c.kda_head_dim
    HD = H * D
    a = dec._norm_act(x, lw.ln1, ACT_FOR_WEIGHT[w.in_qkv.fmt], also_bf16=True, res_only=True)
    x = dec.res(x)
    hb = dec._as_act(a.bf16, "bf16")
    qkv = ops.linear(a, w.in_qkv)                                                    # [T, 3 HD]
    g_raw = ops.linear(dec._as_act(ops.linear(hb, w.f_a), "bf16"), w.f_b, out_f32=True)   # [T, HD]
    b_raw = ops.linear(hb, w.b_proj, out_f32=True)                                   # [T, H]
    o_gate = ops.linear(dec._as_act(ops.linear(hb, w.g_a), "bf16"), w.g_b)           # [T, HD] bf16
    stash = getattr(batch, "spec_stash", None)
    ws = stash is None
    conv_out = rops.causal_conv1d(qkv, 3 * HD, w.conv_w, None, pool.conv[sidx], batch, activation=True, write_state=ws)
    y = rops.kda_recurrence(conv_out, g_raw, b_raw, w.A_log, w.dt_bias, c.kda_gate_lower_bound, pool.ssm[sidx], batch,
                            heads=H, dim=D, write_state=ws, norm=(w.norm_w, o_gate, c.rms_eps))   # bf16 [T, HD]
    if stash is not None:
        stash.layers[sidx] = ("kda", lw, qkv, conv_out, (g_raw, b_raw))
    ya = dec._as_act(y, ACT_FOR_WEIGHT[w.out.fmt])
    return dec.tp.linear_reduce(ya, w.out, residual=x, defer=True)


def _tile(owner, w: torch.Tensor, n: int) -> torch.Tensor:
    """`w` repeated n times (the per-head norm weight laid out for all heads of a row), built once
    and kept on the layer's own weight object: a cache keyed by anything else (a device address,
    say) would outlive the weights and hand a later model another layer's values."""
    t = getattr(owner, "_norm_w_tiled", None)
    if t is None or t.numel() != w.numel() * n or t.device != w.device:
        t = w.repeat(n).contiguous()
        owner._norm_w_tiled = t
    return t


def mamba2_block(dec, x, lw, batch, pool, sidx: int):
    c, w = dec.cfg, lw.mixer
    H, G, P, N = w.heads, w.groups, c.mamba_head_dim, c.mamba_state
    inner, GN = H * P, G * N
    a = dec._norm_act(x, lw.ln1, ACT_FOR_WEIGHT[w.in_proj.fmt], res_only=True)
    x = dec.res(x)
    zxbcdt = ops.linear(a, w.in_proj)                                 # [T, 2 inner + 2GN + H]
    stash = getattr(batch, "spec_stash", None)
    ws = stash is None
    xbc = rops.causal_conv1d(zxbcdt[:, inner:], inner + 2 * GN, w.conv_w, w.conv_b, pool.conv[sidx], batch,
                             activation=True, write_state=ws)
    dt = zxbcdt[:, 2 * inner + 2 * GN:]
    y = rops.mamba2_scan(xbc, dt, w.A_log, w.D, w.dt_bias, pool.ssm[sidx], batch, heads=H, groups=G,
                         head_dim=P, state=N, write_state=ws)          # [T, inner] fp32
    if stash is not None:
        stash.layers[sidx] = ("mamba2", lw, zxbcdt, xbc, dt)
    z = zxbcdt[:, :inner]
    ya = ops.row_op(y, ACT_FOR_WEIGHT[w.out.fmt], ops.IN_GATED_RMSNORM, gate=z, w=w.norm_w,
                    group=inner // max(1, G), eps=c.rms_eps)[0]
    return dec.tp.linear_reduce(ya, w.out, residual=x, defer=True)


def commit_recurrent(cfg, pool, stash, commit_batch) -> None:
    """Advance the state of every recurrent layer by the accepted rows of a verify step:
    `commit_batch` is that step's batch with q_len replaced by the number of rows to commit per
    sequence (0 = leave the sequence's state as it was)."""
    for sidx, (kind, lw, x_in, conv_out, gate) in stash.layers.items():
        w = lw.mixer
        if kind == "gdn":
            kd, vd, kh, vh = cfg.gdn_k_dim, cfg.gdn_v_dim, w.k_heads, w.v_heads
            rops.causal_conv1d(x_in, 2 * kh * kd + vh * vd, w.conv_w, None, pool.conv[sidx], commit_batch,
                               activation=True, write_out=False)
            rops.gdn_recurrence(conv_out, gate, w.A_log, w.dt_bias, pool.ssm[sidx], commit_batch,
                                k_heads=kh, v_heads=vh, k_dim=kd, v_dim=vd, write_out=False)
        elif kind == "kda":
            H, D = w.heads, cfg.kda_head_dim
            rops.causal_conv1d(x_in, 3 * H * D, w.conv_w, None, pool.conv[sidx], commit_batch, activation=True,
                               write_out=False)
            rops.kda_recurrence(conv_out, gate[0], gate[1], w.A_log, w.dt_bias, cfg.kda_gate_lower_bound, pool.ssm[sidx],
                                commit_batch, heads=H, dim=D, write_out=False)
        else:
            H, G, P, N = w.heads, w.groups, cfg.mamba_head_dim, cfg.mamba_state
            inner, GN = H * P, G * N
            rops.causal_conv1d(x_in[:, inner:], inner + 2 * GN, w.conv_w, w.conv_b, pool.conv[sidx], commit_batch,
                               activation=True, write_out=False)
            rops.mamba2_scan(conv_out, gate, w.A_log, w.D, w.dt_bias, pool.ssm[sidx], commit_batch, heads=H,
                             groups=G, head_dim=P, state=N, write_out=False)
