"""CPU checks of the reference op layer: codecs, scale-factor tiling, op semantics."""
import math

import torch

from metrale_inference_alpha_b200 import ops
from metrale_inference_alpha_b200.ops import reference as ref


def test_e2m1_roundtrip_and_ties():
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -1.5, -6.0, 100.0])
    dec = ref.e2m1_decode(ref.e2m1_encode(vals))
    assert torch.equal(dec, torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -1.5, -6.0, 6.0]))
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert torch.equal(ref.e2m1_decode(ref.e2m1_encode(ties)), torch.tensor([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]))


def test_fp4_pack_even_k_low_nibble():
    codes = torch.tensor([[1, 2, 3, 4]], dtype=torch.uint8)
    p = ref.pack_fp4(codes)
    assert p.tolist() == [[0x21, 0x43]]
    assert torch.equal(ref.unpack_fp4(p), codes)


def test_nvfp4_quant_error_bound():
    x = torch.randn(8, 256)
    q, sf, g = ref.quantize_nvfp4(x)
    d = ref.dequantize_nvfp4(q, sf, g)
    rel = (d - x).norm() / x.norm()
    assert rel < 0.12
    wq = ops.make_weight(x, "nvfp4")
    assert (wq.dequant() - x).norm() / x.norm() < 0.12


def test_fp8_quantisers():
    x = torch.randn(300, 260)
    q, s = ref.quantize_fp8_rowwise(x)
    assert ((ref.from_e4m3(q) * s[:, None]) - x).abs().max() < 0.07 * x.abs().max()
    q, s = ref.quantize_fp8_block128(x)
    assert s.shape == (3, 3)
    assert (ref.dequantize_fp8_block128(q, s) - x).abs().max() < 0.07 * x.abs().max()
    q, s = ref.quantize_fp8_group128(x)
    assert s.shape == (3, 300)


def test_sf_tiling_roundtrip_and_offsets():
    sf = torch.randint(0, 255, (200, 12), dtype=torch.uint8)
    t = ref.sf_to_tiled(sf, 4)
    assert t.shape == (2, 4, 512)
    assert torch.equal(ref.tiled_to_sf(t, 200, 12), sf)
    r, kb = 170, 9                       # block 1, row 42 -> r32 10, rq 1; k64 2, kk 1
    assert t[1, 2, 10 * 16 + 1 * 4 + 1] == sf[r, kb]


def test_linear_formats_agree_with_fp32():
    x = torch.randn(6, 512)
    w = torch.randn(64, 512) * 0.05
    want = x @ w.t()
    for fmt, tol in (("bf16", 0.02), ("fp8_row", 0.06), ("fp8_block", 0.06), ("nvfp4", 0.2)):
        a = ops.encode_act_ref(x, ops.ACT_FOR_WEIGHT[fmt])
        y = ops.linear(a, ops.make_weight(w, fmt), out_f32=True)
        assert (y - want).norm() / want.norm() < tol, fmt


def test_swiglu_interleave():
    x = torch.randn(3, 64)
    g, u = torch.randn(16, 64), torch.randn(16, 64)
    w = ops.make_weight(ops.interleave_gate_up(g, u), "bf16")
    y = ops.linear(ops.encode_act_ref(x, "bf16"), w, swiglu=True, out_f32=True)
    xb = ref.bf16_round(x)
    want = torch.nn.functional.silu(xb @ ref.bf16_round(g).t()) * (xb @ ref.bf16_round(u).t())
    assert torch.allclose(y, want, atol=1e-4)


def test_paged_attention_matches_dense():
    torch.manual_seed(0)
    Hq, Hkv, D, bs = 4, 2, 64, 16
    ctx, ql = 40, 5
    k = torch.randn(ctx, Hkv, D)
    v = torch.randn(ctx, Hkv, D)
    q = torch.randn(ql, Hq, D)
    kc = torch.zeros(8, bs, Hkv, D)
    vc = torch.zeros(8, bs, Hkv, D)
    bt = torch.tensor([[5, 2, 7]], dtype=torch.int32)
    slots = torch.tensor([int(bt[0, i // bs]) * bs + i % bs for i in range(ctx)])
    ref.kv_cache_write(kc, vc, k, v, slots)
    out = ref.paged_attention(q, kc, vc, bt, torch.tensor([0]), torch.tensor([ql]), torch.tensor([ctx]),
                              1 / math.sqrt(D))
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    for i in range(ql):
        n = ctx - ql + i + 1
        s = torch.einsum("hd,khd->hk", q[i], kk[:n]) / math.sqrt(D)
        want = torch.einsum("hk,khd->hd", torch.softmax(s, -1), vv[:n])
        assert torch.allclose(out[i], want, atol=1e-5)


def test_rope_neox_partial():
    cos, sin = ref.rope_tables(16, 8, 10000.0)
    x = torch.randn(2, 1, 16)
    y = ref.apply_rope_neox(x, torch.tensor([0, 3]), cos, sin)
    assert torch.allclose(y[0], x[0])                       # position 0 is the identity
    assert torch.equal(y[..., 8:], x[..., 8:])              # channels past rot untouched
    assert torch.allclose(y[1].norm(), x[1].norm(), atol=1e-5)


def test_gdn_and_mamba_steps_shapes_and_decay():
    B, Hk, Hv, Dk, Dv = 2, 2, 4, 8, 16
    h = torch.zeros(B, Hv, Dk, Dv)
    q, k = ref.l2_norm(torch.randn(B, Hk, Dk)), ref.l2_norm(torch.randn(B, Hk, Dk))
    v = torch.randn(B, Hv, Dv)
    g, beta = ref.gdn_gates(torch.randn(B, Hv), torch.randn(B, Hv), torch.zeros(Hv), torch.zeros(Hv))
    o, h1 = ref.gdn_recurrence_step(h, q, k, v, g, beta)
    assert o.shape == (B, Hv, Dv) and h1.shape == h.shape
    # with a zero state, h1 = k (x) (v * beta)
    kk = k.repeat_interleave(2, 1)
    assert torch.allclose(h1, torch.einsum("bhk,bhv->bhkv", kk, v * beta[:, :, None]), atol=1e-6)
    hm = torch.zeros(B, 4, 8, 16)
    y, hm1 = ref.mamba2_step(hm, torch.randn(B, 4, 8), torch.randn(B, 4), torch.zeros(4), torch.randn(B, 2, 16),
                             torch.randn(B, 2, 16), torch.ones(4), torch.zeros(4))
    assert y.shape == (B, 4, 8) and hm1.shape == hm.shape


def test_conv1d_update_window():
    st = torch.zeros(1, 3, 3)
    w = torch.tensor([[0.0, 0.0, 0.0, 1.0]]).repeat(3, 1)
    y, st = ref.causal_conv1d_update(st, torch.tensor([[1.0, 2.0, 3.0]]), w, activation=False)
    assert torch.equal(y, torch.tensor([[1.0, 2.0, 3.0]]))
    assert torch.equal(st[:, :, -1], torch.tensor([[1.0, 2.0, 3.0]]))


def test_routers():
    logits = torch.tensor([[1.0, 3.0, 3.0, 0.0, -1.0, 2.0, 0.5, 0.1]])
    w, idx = ref.route_softmax_topk(logits, 2)
    assert idx.tolist() == [[1, 2]] and abs(float(w.sum()) - 1) < 1e-6
    w, idx = ref.route_sigmoid_grouped(logits, torch.zeros(8), 2, n_group=4, topk_group=1)
    assert idx.tolist() == [[2, 3]] or idx.tolist() == [[1, 0]] or set(idx[0].tolist()) <= {2, 3}


def test_sampler_reference_greedy_and_topk():
    x = torch.tensor([[0.0, 5.0, 1.0, 4.9]])
    one = lambda v, dt=torch.float32: torch.tensor([v], dtype=dt)
    ids, _ = ops.sample(x, one(0.0), one(0, torch.int32), one(1.0), one(0.0), one(1, torch.int64), one(0, torch.int64))
    assert ids.tolist() == [1]
    for s in range(20):
        ids, _ = ops.sample(x, one(1.0), one(2, torch.int32), one(1.0), one(0.0), one(s, torch.int64), one(0, torch.int64))
        assert ids.item() in (1, 3)


def test_rope_scaling_tables_match_transformers():
    """linear / llama3 / yarn inverse frequencies and attention factor against the HF oracle."""
    from types import SimpleNamespace
    import torch
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    from metrale_inference_alpha_b200.ops import reference as ref
    cases = [
        {"rope_type": "linear", "factor": 4.0},
        {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
         "original_max_position_embeddings": 8192},
        {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768},
        {"rope_type": "yarn", "factor": 40.0, "original_max_position_embeddings": 4096, "beta_fast": 32, "beta_slow": 1,
         "mscale": 1.0, "mscale_all_dim": 1.0},
    ]
    for sc in cases:
        theta, D = 1e6, 128
        cfg = SimpleNamespace(rope_theta=theta, head_dim=D, hidden_size=D * 8, num_attention_heads=8,
                              partial_rotary_factor=1.0, max_position_embeddings=131072, rope_scaling=dict(sc),
                              rope_parameters=dict(sc, rope_theta=theta))
        cfg.standardize_rope_params = lambda: None
        try:
            want, att = ROPE_INIT_FUNCTIONS[sc["rope_type"]](cfg, device="cpu")
        except Exception as e:                      # signature drift between transformers versions
            import pytest
            pytest.skip(f"transformers oracle unavailable: {e}")
        got, att_got = ref.rope_inv_freq(D, theta, sc)
        assert torch.allclose(got.float(), want.float(), rtol=1e-5, atol=1e-9), sc
        assert abs(att_got - float(att)) < 1e-6, sc
    cos, sin = ref.rope_tables(64, 128, 1e6, scaling={"rope_type": "linear", "factor": 2.0})
    c0, s0 = ref.rope_tables(64, 128, 1e6)
    assert torch.allclose(cos[2 * 7], c0[7], atol=1e-6) and torch.allclose(sin[2 * 7], s0[7], atol=1e-6)
