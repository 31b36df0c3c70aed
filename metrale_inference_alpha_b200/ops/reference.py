"""Plain PyTorch restatement of every op in the engine (fp32 math, any device).

This module is the numerical oracle for the CUDA kernels and the execution path on CPU.
Formulas follow the reference's kernel headers (file:line cited per function, paths
relative to the reference tree).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

F8 = torch.float8_e4m3fn
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


# ----------------------------------------------------------------------------- fp8 / fp4 codecs
def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 bytes (uint8), round-to-nearest-even, saturating at +-448."""
    return x.float().clamp(-448.0, 448.0).to(F8).view(torch.uint8)


def from_e4m3(b: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes -> fp32. The NaN code reads as 0 (kernels/gb10/common/dequant_nvfp4_bf16.cu:2-15)."""
    f = b.view(F8).float()
    return torch.nan_to_num(f, nan=0.0)


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit e2m1 codes (uint8 0..15), RNE on {0,.5,1,1.5,2,3,4,6}, saturating."""
    a = x.abs()
    c = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
         + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8)
         + (a > 5.0).to(torch.uint8))
    return c | ((x < 0).to(torch.uint8) << 3)


def e2m1_decode(c: torch.Tensor) -> torch.Tensor:
    mag = E2M1_VALUES.to(c.device)[(c & 7).long()]
    return torch.where((c & 8) != 0, -mag, mag)


def pack_fp4(codes: torch.Tensor) -> torch.Tensor:
    """[.., K] codes -> [.., K/2] bytes, even k in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).flatten(-2)


def quantize_nvfp4(x: torch.Tensor, per_row_global: bool = True, static_scale: float = 0.0):
    """x [R, K] -> (packed [R, K/2] u8, sf [R, K/16] u8 e4m3, global [R] or scalar fp32).

    global = amax / (6 * 448); block scale = e4m3(blockmax / (6 * global))
    (kernels/gb10/common/quantize_bf16_to_nvfp4.cu:2-16, per-row variant of scale2)."""
    x = x.float()
    R, K = x.shape
    assert K % 16 == 0
    amax = x.abs().amax(dim=1) if per_row_global else x.abs().amax().expand(R)
    gs = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax))
    if static_scale > 0:                       # calibrated global scale (ModelOpt `input_scale` semantics)
        gs = torch.full_like(gs, float(static_scale))
    xb = x.view(R, K // 16, 16)
    bmax = xb.abs().amax(dim=2)
    sf = to_e4m3(bmax / (6.0 * gs[:, None]))
    sff = from_e4m3(sf)
    inv = torch.where(sff > 0, 1.0 / (sff * gs[:, None]), torch.zeros_like(sff))
    codes = e2m1_encode(xb * inv[:, :, None]).view(R, K)
    g = gs if per_row_global else gs[0]
    return pack_fp4(codes), sf, g


def dequantize_nvfp4(packed, sf, gscale) -> torch.Tensor:
    """w = E2M1(nibble) * E4M3(scale) * global (kernels/gb10/common/dequant_nvfp4_bf16.cu:2-15)."""
    vals = e2m1_decode(unpack_fp4(packed))
    R, K = vals.shape
    g = gscale if torch.is_tensor(gscale) else torch.tensor(gscale)
    g = g.float().to(vals.device)
    g = g.view(-1, 1, 1) if g.ndim >= 1 and g.numel() > 1 else g.reshape(1, 1, 1)
    return (vals.view(R, K // 16, 16) * from_e4m3(sf)[:, :, None] * g).view(R, K)


def quantize_fp8_rowwise(x: torch.Tensor):
    """x [R, K] -> (e4m3 bytes [R, K], scale [R]) with scale = amax / 448."""
    x = x.float()
    amax = x.abs().amax(dim=1)
    sc = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    return to_e4m3(x * (1.0 / sc)[:, None]), sc


def quantize_fp8_group128(x: torch.Tensor):
    """Activation quantiser: one scale per row per 128 channels; scales returned [K/128, R]."""
    x = x.float()
    R, K = x.shape
    G = (K + 127) // 128
    pad = G * 128 - K
    xp = torch.nn.functional.pad(x, (0, pad)).view(R, G, 128)
    amax = xp.abs().amax(dim=2)
    sc = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = to_e4m3(xp * (1.0 / sc)[:, :, None]).view(R, G * 128)[:, :K]
    return q.contiguous(), sc.t().contiguous()


def quantize_fp8_block128(w: torch.Tensor):
    """Weight quantiser: w[n,k] = e4m3[n,k] * scale[n/128, k/128]
    (crates/model-layers/src/weight_map/loaders_fp8.rs:18-60)."""
    w = w.float()
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.nn.functional.pad(w, (0, kb * 128 - K, 0, nb * 128 - N)).view(nb, 128, kb, 128)
    amax = wp.abs().amax(dim=(1, 3))
    sc = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = to_e4m3(wp / sc[:, None, :, None]).view(nb * 128, kb * 128)[:N, :K]
    return q.contiguous(), sc


def dequantize_fp8_block128(q: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    s = sc.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return from_e4m3(q) * s


def sf_to_tiled(sf: torch.Tensor, sf_k64: Optional[int] = None) -> torch.Tensor:
    """Row-major ue4m3 scale factors [R, K/16] -> the 128x4 tiled layout the tensor core's
    scale-factor copy consumes: [ceil(R/128), sf_k64, 512] with byte offset
    (r % 32) * 16 + (r // 32 % 4) * 4 + k4 inside a tile. Zero padded."""
    R, KB = sf.shape
    k64 = (KB + 3) // 4
    sf_k64 = sf_k64 or k64
    nb = (R + 127) // 128
    buf = torch.zeros(nb * 128, sf_k64 * 4, dtype=torch.uint8, device=sf.device)
    buf[:R, :KB] = sf
    t = buf.view(nb, 4, 32, sf_k64, 4)            # [nb, rq, r32, k64, kk]
    return t.permute(0, 3, 2, 1, 4).contiguous().view(nb, sf_k64, 512)


def tiled_to_sf(t: torch.Tensor, R: int, KB: int) -> torch.Tensor:
    nb, sf_k64, _ = t.shape
    x = t.view(nb, sf_k64, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(nb * 128, sf_k64 * 4)
    return x[:R, :KB].contiguous()


# ----------------------------------------------------------------------------- norms / activations
def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def rms_norm(x, w, eps: float, plus_one: bool = False):
    """FP32 math; `(1 + weight)` scaling when plus_one (kernels/gb10/common/rms_norm.cu:3-8)."""
    x = x.float()
    inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    ww = w.float() + 1.0 if plus_one else w.float()
    return x * inv * ww


def gated_rms_norm(x, gate, w, eps: float, group: int = 0):
    """out = x * rsqrt(mean(x^2)+eps) * w * silu(gate), statistics per `group` channels
    (kernels/gb10/common/rms_norm.cu:1099-1172)."""
    x = x.float()
    K = x.shape[-1]
    G = group or K
    xs = x.view(*x.shape[:-1], K // G, G)
    inv = torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps)
    y = (xs * inv).view_as(x) * w.float()
    if gate is not None:
        y = y * torch.nn.functional.silu(gate.float())
    return y


def l2_norm(x, eps: float = 1e-6):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return torch.nn.functional.silu(g) * u


def relu2(x: torch.Tensor) -> torch.Tensor:
    return torch.relu(x.float()).pow(2)


# ----------------------------------------------------------------------------- rope
def rope_inv_freq(rot: int, theta: float, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, float]:
    """Inverse frequencies [rot/2] (float64) and the attention factor that multiplies cos / sin, for
    the plain table and the long-context rescalings of HF `rope_scaling` configs: linear (position
    interpolation), llama3 (low / high frequency bands), yarn (NTK-by-parts + mscale). The kernels
    only ever see the finished tables, so every variant costs nothing at run time
    (kernels/gb10/common/rope.cu: rope_forward, rope_yarn, rope_proportional)."""
    import math
    inv = theta ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)
    if not scaling:
        return inv, 1.0
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    factor = float(scaling.get("factor", 1.0))
    if kind in ("default", None):
        return inv, 1.0
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        mid = (1 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > old / lo, inv / factor, torch.where(wavelen < old / hi, inv, mid))
        return out, 1.0
    if kind == "yarn":
        old = float(scaling.get("original_max_position_embeddings", 4096))
        beta_fast, beta_slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

        def get_mscale(scale, m=1.0):
            return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0
        ms, ms_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
        att = scaling.get("attention_factor")
        if att is None:
            att = get_mscale(factor, ms) / get_mscale(factor, ms_all) if (ms and ms_all) else get_mscale(factor)

        def corr_dim(n_rot):
            return (rot * math.log(old / (n_rot * 2 * math.pi))) / (2 * math.log(theta))
        low, high = corr_dim(beta_fast), corr_dim(beta_slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, rot - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rot // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        extrap_w = 1 - ramp                                      # 1 = keep the original frequency
        return (inv / factor) * (1 - extrap_w) + inv * extrap_w, float(att)
    raise ValueError(f"unsupported rope_scaling type {kind!r}")


def rope_tables(max_pos: int, rot: int, theta: float, device="cpu", scaling: Optional[dict] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [max_pos, rot/2] with freq_i = theta^(-2i/rot) (kernels/gb10/common/rope.cu:11-21),
    optionally rescaled for long context (see rope_inv_freq)."""
    inv, att = rope_inv_freq(rot, theta, scaling)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return (ang.cos() * att).float().to(device), (ang.sin() * att).float().to(device)


def apply_rope_neox(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """x [T, H, D]; pairs (i, i + rot/2); channels past rot untouched."""
    x = x.float()
    half = cos.shape[1]
    c = cos[positions.long()][:, None, :]
    s = sin[positions.long()][:, None, :]
    x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


# ----------------------------------------------------------------------------- paged attention
def kv_cache_write(k_cache, v_cache, k, v, slots, k_scale=None, v_scale=None):
    """Scatter rows into caches [num_blocks, block, Hkv, D] by flat slot; e4m3 caches store
    value / scale (stored scale is the dequant multiplier, kv_scale_keys.rs:1-60)."""
    nb, bs, H, D = k_cache.shape
    kf, vf = k_cache.view(nb * bs, H, D), v_cache.view(nb * bs, H, D)
    ok = slots >= 0
    idx = slots[ok].long()
    if k_cache.dtype == torch.uint8:
        kf[idx] = to_e4m3(k.float()[ok] * (1.0 / k_scale))
        vf[idx] = to_e4m3(v.float()[ok] * (1.0 / v_scale))
    else:
        kf[idx] = k[ok].to(k_cache.dtype)
        vf[idx] = v[ok].to(v_cache.dtype)


def paged_attention(q, k_cache, v_cache, block_table, q_start, q_len, ctx_len, scale: float,
                    k_scale=None, v_scale=None, window: int = 0) -> torch.Tensor:
    """Causal attention of each sequence's `q_len` new query rows over its `ctx_len` cached
    tokens (the new tokens are the last q_len of them). q [T, Hq, D] -> out [T, Hq, D] fp32."""
    T, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    G = Hq // Hkv
    out = torch.zeros(T, Hq, D, dtype=torch.float32, device=q.device)
    for s in range(len(q_len)):
        ql, ctx, qs = int(q_len[s]), int(ctx_len[s]), int(q_start[s])
        if ql <= 0:
            continue
        nblk = (ctx + bs - 1) // bs
        blocks = block_table[s, :nblk].long()
        kk = k_cache[blocks].reshape(nblk * bs, Hkv, -1)[:ctx]
        vv = v_cache[blocks].reshape(nblk * bs, Hkv, -1)[:ctx]
        if k_cache.dtype == torch.uint8:
            kk = from_e4m3(kk) * k_scale
            vv = from_e4m3(vv) * v_scale
        kk, vv = kk.float(), vv.float()
        qq = q[qs:qs + ql].float()                                   # [ql, Hq, D]
        kk = kk.repeat_interleave(G, dim=1)                          # [ctx, Hq, D]
        vv = vv.repeat_interleave(G, dim=1)
        sc = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        pos_q = torch.arange(ctx - ql, ctx, device=q.device)[:, None]
        pos_k = torch.arange(ctx, device=q.device)[None, :]
        mask = pos_k <= pos_q
        if window > 0:
            mask &= pos_k > pos_q - window
        sc = sc.masked_fill(~mask[None], float("-inf"))
        p = torch.softmax(sc, dim=-1)
        out[qs:qs + ql] = torch.einsum("hqk,khd->qhd", p, vv)
    return out


# ----------------------------------------------------------------------------- gated delta net
def gdn_gates(a, b, A_log, dt_bias):
    """decay = exp(-exp(min(A_log,20)) * softplus(min(a+dt_bias,20))), beta = sigmoid(b)
    (kernels/gb10/common/ssm_preprocess.cu:10-12,576-616)."""
    sp = torch.log1p(torch.exp(torch.clamp(a.float() + dt_bias.float(), max=20.0)))
    decay = torch.exp(-torch.exp(torch.clamp(A_log.float(), max=20.0)) * sp)
    return decay, torch.sigmoid(b.float())


def gdn_recurrence_step(h, q, k, v, g, beta):
    """One token. h [B, Hv, Dk, Dv] fp32; q,k [B, Hk, Dk]; v [B, Hv, Dv]; g,beta [B, Hv].
    v' = (v - g*(h^T k)) * beta; h = g*h + k (x) v'; out = h^T q / sqrt(Dk)
    (kernels/gb10/common/gated_delta_rule.cu:8-16). Returns (out [B,Hv,Dv], h)."""
    B, Hv, Dk, Dv = h.shape
    rep = Hv // k.shape[1]
    kk = k.float().repeat_interleave(rep, dim=1)
    qq = q.float().repeat_interleave(rep, dim=1)
    gg = g.float()[:, :, None, None]
    hk = torch.einsum("bhkv,bhk->bhv", h, kk)
    vp = (v.float() - g.float()[:, :, None] * hk) * beta.float()[:, :, None]
    h = gg * h + torch.einsum("bhk,bhv->bhkv", kk, vp)
    out = torch.einsum("bhkv,bhk->bhv", h, qq) / math.sqrt(Dk)
    return out, h


def causal_conv1d_update(state, x, w, bias=None, activation: bool = True):
    """state [B, C, d-1] fp32 (oldest first), x [B, C] new column, w [C, d] (tap 0 = oldest).
    y = SiLU(bias + sum_k win[k] * w[:, k]) (kernels/gb10/common/causal_conv1d.cu:2-10).
    Returns (y [B, C], new state)."""
    win = torch.cat([state.float(), x.float()[:, :, None]], dim=2)
    y = (win * w.float()[None]).sum(-1)
    if bias is not None:
        y = y + bias.float()
    if activation:
        y = torch.nn.functional.silu(y)
    return y, win[:, :, 1:].contiguous()


# ----------------------------------------------------------------------------- mamba2
def mamba2_step(h, x, dt, A_log, B, Cm, Dp, dt_bias, dt_min: float = 0.0, dt_max: float = float("inf")):
    """Selective scan, one token. h [Bt, H, P, N] fp32; x [Bt, H, P]; dt [Bt, H]; B, Cm [Bt, G, N].
    dt = clamp(softplus(dt + bias)); dA = exp(-exp(A_log) dt); h = dA h + dt x (x) B; y = h C + D x
    (kernels/gb10/common/mamba2_ssm_decode.cu:7-20)."""
    Bt, H, P, N = h.shape
    G = B.shape[1]
    rep = H // G
    dtv = torch.nn.functional.softplus(dt.float() + dt_bias.float()).clamp(dt_min, dt_max)
    dA = torch.exp(-torch.exp(A_log.float()) * dtv)
    Bh = B.float().repeat_interleave(rep, dim=1)
    Ch = Cm.float().repeat_interleave(rep, dim=1)
    h = dA[:, :, None, None] * h + (dtv[:, :, None] * x.float())[:, :, :, None] * Bh[:, :, None, :]
    y = torch.einsum("bhpn,bhn->bhp", h, Ch) + Dp.float()[None, :, None] * x.float()
    return y, h


# ----------------------------------------------------------------------------- MoE routing
def route_softmax_topk(logits: torch.Tensor, k: int, renormalize: bool = True):
    """softmax over experts, top-k, ties -> lower index (kernels/gb10/common/moe_topk.cu)."""
    p = torch.softmax(logits.float(), dim=-1)
    w, idx = _topk_stable(p, k)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


def route_sigmoid_grouped(logits, bias, k: int, n_group: int = 1, topk_group: int = 1,
                          renormalize: bool = True, scaling: float = 1.0):
    """sigmoid scores; selection uses score + bias; group-limited: keep the `topk_group` groups
    with the largest sum of their top-2 biased scores, then top-k inside them; weights are
    the un-biased scores, sum-normalised, times `scaling`
    (kernels/gb10/common/moe_topk_sigmoid.cu header for the un-grouped form; grouping follows
    the DeepSeek-V3 router)."""
    s = torch.sigmoid(logits.float())
    sel = s + (bias.float() if bias is not None else 0.0)
    T, E = sel.shape
    if n_group > 1:
        gs = sel.view(T, n_group, E // n_group)
        gscore = gs.topk(2, dim=-1).values.sum(-1)
        _, gidx = _topk_stable(gscore, topk_group)
        gmask = torch.zeros(T, n_group, dtype=torch.bool, device=sel.device)
        gmask.scatter_(1, gidx, True)
        sel = sel.masked_fill(~gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E),
                              float("-inf"))
    _, idx = _topk_stable(sel, k)
    w = s.gather(1, idx)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scaling, idx


def _topk_stable(x: torch.Tensor, k: int):
    """top-k with ties resolved toward the lower index."""
    order = torch.sort(x, dim=-1, descending=True, stable=True)
    return order.values[..., :k], order.indices[..., :k]


# ----------------------------------------------------------------------------- MXFP4 (OCP microscaling)
def e8m0_to_float(b: torch.Tensor) -> torch.Tensor:
    """E8M0 block scales: 2 ** (byte - 127); byte 255 is NaN."""
    e = b.to(torch.int32)
    out = torch.pow(2.0, (e - 127).float())
    return torch.where(e == 255, torch.full_like(out, float("nan")), out)


def dequantize_mxfp4(packed: torch.Tensor, scales_e8m0: torch.Tensor) -> torch.Tensor:
    """MXFP4 weights (e2m1 values, two per byte with the low nibble first, one E8M0 scale per 32
    values along K) -> fp32 [N, K]. Host-side unpack used to convert MXFP4 checkpoints to a serving
    format (role of the reference's crates/core/src/mxfp4_e8m0.rs)."""
    N, kb = packed.shape
    K = kb * 2
    assert scales_e8m0.shape == (N, K // 32), "one E8M0 scale per 32 values"
    vals = e2m1_decode(unpack_fp4(packed))                     # [N, K] fp32
    s = e8m0_to_float(scales_e8m0).repeat_interleave(32, dim=1)
    return vals * s


# ----------------------------------------------------------------------------- Kimi delta attention
def kda_gate(g_raw, A_log, dt_bias, lower_bound: float):
    """Bounded per-channel log-decay: lower_bound * sigmoid(exp(A_log[h]) * (g_raw[t,h,d] + dt_bias[h,d]))
    (kernels/gb10/common/kda_gate.cu). g_raw [T, H, D] -> fp32 [T, H, D] in (lower_bound, 0)."""
    a = torch.exp(torch.clamp(A_log.float(), max=20.0))[None, :, None]
    return lower_bound * torch.sigmoid(a * (g_raw.float() + dt_bias.float().view(1, *g_raw.shape[1:])))


def kda_recurrence_step(S, q, k, v, gate, beta):
    """One token of the per-channel gated delta rule (kernels/gb10/common/kda_recurrent.cu). S [B, H, D, D]
    fp32 indexed [k][v]; q, k already l2-normalised, v, gate (log-decay) [B, H, D]; beta [B, H] already
    sigmoided. Returns (out [B, H, D], S)."""
    D = S.shape[-1]
    S = S * torch.exp(gate.float())[..., None]
    delta = (v.float() - torch.einsum("bhkv,bhk->bhv", S, k.float())) * beta.float()[..., None]
    S = S + torch.einsum("bhk,bhv->bhkv", k.float(), delta)
    return torch.einsum("bhkv,bhk->bhv", S, q.float()) / math.sqrt(D), S


def kda_chunk(S, q, k, v, gate, beta, chunk: int = 32):
    """The same recurrence over T tokens of one sequence in chunks (the WY / UT-transform form of
    kernels/gb10/common/kda_chunk.cu): q, k, v, gate [T, H, D], beta [T, H], S [H, D, D]. Used as a
    second oracle: it must agree with T applications of `kda_recurrence_step`."""
    T, H, D = q.shape
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros(T, H, D)
    S = S.clone().float()
    for c0 in range(0, T, chunk):
        C = min(chunk, T - c0)
        qc, kc, vc = (x[c0:c0 + C].float().transpose(0, 1) for x in (q, k, v))           # [H, C, D]
        gc = gate[c0:c0 + C].float().transpose(0, 1).cumsum(1)                             # [H, C, D]
        bc = beta[c0:c0 + C].float().transpose(0, 1)                                        # [H, C]
        kd = kc[:, :, None, :] * kc[:, None, :, :] * torch.exp(gc[:, :, None, :] - gc[:, None, :, :])
        A = -(bc[:, :, None] * kd.sum(-1)).tril(-1)                                         # [H, C, C]
        for i in range(1, C):
            A[:, i, :i] = A[:, i, :i] + torch.einsum("hj,hjm->hm", A[:, i, :i], A[:, :i, :i])
        A = A + torch.eye(C)
        u = A @ (vc * bc[..., None])
        w = A @ (kc * bc[..., None] * torch.exp(gc))
        v_new = u - w @ S
        intra = ((qc[:, :, None, :] * kc[:, None, :, :] * torch.exp(gc[:, :, None, :] - gc[:, None, :, :])).sum(-1) * scale).tril(0)
        o = scale * (qc * torch.exp(gc)) @ S + intra @ v_new
        last = gc[:, -1:, :]
        S = S * torch.exp(last).transpose(1, 2) + (kc * torch.exp(last - gc)).transpose(1, 2) @ v_new
        out[c0:c0 + C] = o.transpose(0, 1)
    return out, S


def sigmoid_gated_rmsnorm(x, gate, w, eps: float):
    """x [.., D] fp32: x * rsqrt(mean(x^2) + eps) * w * sigmoid(gate) (kda_layer_ops.cu::kda_o_norm_gated)."""
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float() * torch.sigmoid(gate.float())
