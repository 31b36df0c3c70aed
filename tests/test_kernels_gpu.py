"""Numerics of every CUDA kernel against the plain PyTorch fp32 reference of the same op.
The reference consumes the *same quantised operands*, so tolerances only cover accumulation
order and the final bf16 rounding."""
import math

import pytest
import torch

from metrale_inference_alpha_b200 import ops
from metrale_inference_alpha_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, rtol=2e-2, atol=2e-2):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{bad}/{got.numel()} off; max err {err.max():.4g} (ref max {want.abs().max():.4g})"


def _mk(M, N, K, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.05
    return x, w


def _run_linear(fmt, M, N, K, **kw):
    x, w = _mk(M, N, K)
    qw_cpu = ops.make_weight(w, fmt)
    act_cpu = ops.encode_act_ref(x, ops.ACT_FOR_WEIGHT[fmt])
    want = act_cpu.data @ qw_cpu.dequant().t()
    qw = qw_cpu.to(DEV)
    act = ops.quantize_act(x.to(DEV).to(torch.bfloat16), ops.ACT_FOR_WEIGHT[fmt])
    # the oracle quantises the bf16-rounded activations exactly like the kernel did
    act_cpu = ops.encode_act_ref(x.to(torch.bfloat16).float(), ops.ACT_FOR_WEIGHT[fmt])
    want = act_cpu.data @ qw_cpu.dequant().t()
    got = ops.linear(act, qw, out_f32=True, **kw)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    _close(got, want, rtol=1e-2, atol=1e-2 * want.abs().max().item())
    return got, want


@pytest.mark.parametrize("M", [1, 16, 24, 48, 64, 77, 128, 300])
def test_gemm_bf16(M):
    _run_linear("bf16", M, 384, 512)


def test_gemm_bf16_ragged_n_and_splitk():
    _run_linear("bf16", 40, 200, 1024)                 # N not a multiple of 128
    _run_linear("bf16", 40, 256, 2048, force_splits=4)
    _run_linear("bf16", 130, 256, 2048, force_splits=3)


@pytest.mark.parametrize("M", [1, 18, 24, 32, 33, 128, 260])
def test_gemm_fp8_row(M):
    _run_linear("fp8_row", M, 256, 1024)


@pytest.mark.parametrize("M", [1, 20, 64, 150])
def test_gemm_fp8_block(M):
    _run_linear("fp8_block", M, 384, 1024)
    _run_linear("fp8_block", M, 256, 2048, force_splits=2)


@pytest.mark.parametrize("M", [1, 7, 16, 18, 32, 64, 128, 200])
def test_gemm_nvfp4(M):
    _run_linear("nvfp4", M, 256, 1024)


def test_gemm_splitk_workspace_path_matches_cluster_path():
    for fmt in ("nvfp4", "bf16", "fp8_block"):
        _run_linear(fmt, 24, 384, 2048, force_splits=4, no_cluster=True)
        _run_linear(fmt, 100, 256, 4096, force_splits=3, no_cluster=True)
        _run_linear(fmt, 100, 256, 4096, force_splits=3)
        _run_linear(fmt, 128, 512, 4096, force_splits=8)


@pytest.mark.parametrize("fmt", ["nvfp4", "bf16", "fp8_row"])
@pytest.mark.parametrize("M", [1, 16, 100, 128])
def test_gemm_cluster_splitk_exchange_paths_agree_bitwise(fmt, M):
    """A split-K cluster exchanges its fp32 partial tiles through the L2-resident workspace by
    default and over distributed shared memory on request; both sum in split order, so the
    results are identical, with and without a residual."""
    g = torch.Generator().manual_seed(31)
    N, K = 640, 4096
    qw = ops.make_weight(torch.randn(N, K, generator=g) * 0.05, fmt).to(DEV)
    act = ops.quantize_act(torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV), ops.ACT_FOR_WEIGHT[fmt])
    res = torch.randn(M, N, generator=g).to(torch.bfloat16).to(DEV)
    for splits in (2, 4, 8):
        a = ops.linear(act, qw, residual=res, force_splits=splits)
        b = ops.linear(act, qw, residual=res, force_splits=splits, dsmem_splitk=True)
        c = ops.linear(act, qw, residual=res, force_splits=splits, no_cluster=True)
        torch.cuda.synchronize()
        assert torch.equal(a, b) and torch.equal(a, c), (fmt, M, splits)
    ops.check_status(DEV)
    _run_linear(fmt, M, 384, 2048, force_splits=4)


def test_gemm_nvfp4_splitk_and_tn():
    _run_linear("nvfp4", 24, 384, 2048, force_splits=4)
    _run_linear("nvfp4", 24, 128, 512, force_tn=128)
    _run_linear("nvfp4", 128, 5120, 1024)


def test_gemm_swiglu_and_residual():
    M, I, K = 50, 192, 512
    x, wg = _mk(M, I, K, 1)
    _, wu = _mk(M, I, K, 2)
    w = ops.interleave_gate_up(wg, wu)
    for fmt in ("bf16", "nvfp4", "fp8_row"):
        qw_cpu = ops.make_weight(w, fmt)
        xb = x.to(torch.bfloat16)
        a_cpu = ops.encode_act_ref(xb.float(), ops.ACT_FOR_WEIGHT[fmt])
        want = ops.linear(a_cpu, qw_cpu, swiglu=True, out_f32=True)
        a = ops.quantize_act(xb.to(DEV), ops.ACT_FOR_WEIGHT[fmt])
        got = ops.linear(a, qw_cpu.to(DEV), swiglu=True)
        _close(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    res = torch.randn(M, 2 * I).to(torch.bfloat16)
    qw_cpu = ops.make_weight(w, "bf16")
    a_cpu = ops.encode_act_ref(x.to(torch.bfloat16).float(), "bf16")
    want = ops.linear(a_cpu, qw_cpu, residual=res, out_f32=True)
    got = ops.linear(ops.quantize_act(x.to(torch.bfloat16).to(DEV), "bf16"), qw_cpu.to(DEV),
                     residual=res.to(DEV))
    _close(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    ops.check_status(DEV)


# N / 128 > 148 SMs selects the persistent kernel (tile loop per CTA, two TMEM accumulators)
@pytest.mark.parametrize("fmt", ["nvfp4", "fp8_row", "bf16"])
@pytest.mark.parametrize("M", [1, 16, 50, 128])
def test_gemm_persistent_path_matches_oracle(fmt, M):
    N = 128 * 150 + (64 if fmt == "bf16" else 0)          # bf16 case ends in a ragged tile
    _run_linear(fmt, M, N, 512)


def test_gemm_persistent_matches_one_tile_per_cta_kernel_bitwise():
    M, N, K = 96, 128 * 300, 1024
    x, w = _mk(M, N, K, 5)
    for fmt in ("nvfp4", "fp8_row"):
        qw = ops.make_weight(w, fmt).to(DEV)
        act = ops.quantize_act(x.to(DEV).to(torch.bfloat16), ops.ACT_FOR_WEIGHT[fmt])
        a = ops.linear(act, qw)
        b = ops.linear(act, qw, one_tile_per_cta=True)
        assert torch.equal(a, b)
    ops.check_status(DEV)


def test_gemm_persistent_swiglu_and_residual():
    M, I, K = 70, 64 * 160, 512
    x, wg = _mk(M, I, K, 1)
    _, wu = _mk(M, I, K, 2)
    w = ops.interleave_gate_up(wg, wu)
    for fmt in ("nvfp4", "fp8_row", "bf16"):
        qw_cpu = ops.make_weight(w, fmt)
        xb = x.to(torch.bfloat16)
        want = ops.linear(ops.encode_act_ref(xb.float(), ops.ACT_FOR_WEIGHT[fmt]), qw_cpu, swiglu=True, out_f32=True)
        got = ops.linear(ops.quantize_act(xb.to(DEV), ops.ACT_FOR_WEIGHT[fmt]), qw_cpu.to(DEV), swiglu=True)
        _close(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    res = torch.randn(M, 2 * I).to(torch.bfloat16)
    qw_cpu = ops.make_weight(w, "bf16")
    want = ops.linear(ops.encode_act_ref(x.to(torch.bfloat16).float(), "bf16"), qw_cpu, residual=res, out_f32=True)
    got = ops.linear(ops.quantize_act(x.to(torch.bfloat16).to(DEV), "bf16"), qw_cpu.to(DEV), residual=res.to(DEV))
    _close(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    ops.check_status(DEV)


@pytest.mark.parametrize("M", [129, 300, 512])
def test_gemm_persistent_prefill_tiles_match_the_one_tile_per_cta_kernel(M, monkeypatch):
    """Several 128-token tiles on the persistent kernel (work items walk token tiles fastest, the
    activation scales are reloaded per tile): bit-identical to the one-tile-per-CTA kernel, plain,
    with a residual and through the SwiGLU epilogue; ragged last token tile and ragged last weight tile."""
    monkeypatch.setattr(ops, "_PERSIST_PREFILL", 128)
    N, K = 128 * 80 + 64, 768
    x, w = _mk(M, N, K, 11)
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(DEV)
    for fmt in ("nvfp4", "fp8_row", "bf16"):
        if fmt == "nvfp4":
            qw = ops.make_weight(w[:128 * 80], fmt).to(DEV)       # NVFP4 scale tiles want whole 128-row weight tiles
            r = res[:, :128 * 80].contiguous()
        else:
            qw, r = ops.make_weight(w, fmt).to(DEV), res
        act = ops.quantize_act(x.to(DEV).to(torch.bfloat16), ops.ACT_FOR_WEIGHT[fmt])
        a = ops.linear(act, qw, residual=r)
        b = ops.linear(act, qw, residual=r, one_tile_per_cta=True)
        assert torch.equal(a, b), fmt
        assert torch.equal(ops.linear(act, qw), ops.linear(act, qw, one_tile_per_cta=True)), fmt
    I = 64 * 160
    _, wg = _mk(M, I, K, 1)
    _, wu = _mk(M, I, K, 2)
    wi = ops.interleave_gate_up(wg, wu)
    for fmt in ("nvfp4", "bf16"):
        qw = ops.make_weight(wi, fmt).to(DEV)
        act = ops.quantize_act(x.to(DEV).to(torch.bfloat16), ops.ACT_FOR_WEIGHT[fmt])
        got, want = ops.linear(act, qw, swiglu=True), ops.linear(act, qw, swiglu=True, one_tile_per_cta=True)
        # the two epilogues multiply the scales in a different order: equal to a bf16 rounding step
        _close(got, want.float().cpu(), rtol=1e-2, atol=1e-2 * want.float().abs().max().item())
    ops.check_status(DEV)


def _dequant_act(act):
    """NVFP4 activation on the device -> fp32 matrix on the CPU."""
    nb = (act.M + 127) // 128
    sf = ref.tiled_to_sf(act.sf.cpu().view(nb, act.sf_k64, 512), act.M, act.K // 16)
    return ref.dequantize_nvfp4(act.data.cpu(), sf, act.scale.cpu())


@pytest.mark.parametrize("M", [1, 16, 77, 128])
def test_gemm_swiglu_epilogue_quantises_to_nvfp4_with_a_static_scale(M):
    """The persistent kernel's SwiGLU epilogue writes packed e2m1 + tiled ue4m3 scale factors for
    the down projection. Checked against (a) the row kernel quantising the kernel's own bf16
    SwiGLU output with the same static scale and (b) the down projection fed with either."""
    I, K = 64 * 160, 512                                # 160 tiles -> persistent path; I % 256 == 0
    x, wg = _mk(M, I, K, 1)
    _, wu = _mk(M, I, K, 2)
    _, wd = _mk(M, 384, I, 3)
    w = ops.make_weight(ops.interleave_gate_up(wg, wu), "nvfp4").to(DEV)
    down = ops.make_weight(wd, "nvfp4").to(DEV)
    a = ops.quantize_act(x.to(DEV).to(torch.bfloat16), "nvfp4")
    y = ops.linear(a, w, swiglu=True)                   # bf16, unfused
    gs = float(y.float().abs().max()) * 1.5 / (6 * 448)
    fused = ops.linear(a, w, swiglu=True, quant_out=gs)
    unfused = ops.quantize_act(y, "nvfp4", static_scale=gs)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert fused.fmt == "nvfp4" and fused.K == I and torch.all(fused.scale == gs)
    df, du = _dequant_act(fused), _dequant_act(unfused)
    # the fused path quantises the fp32 value, the unfused one its bf16 rounding: a few codes flip
    same = (df == du).float().mean().item()
    assert same > 0.97, same
    assert (df - du).abs().max().item() <= 0.51 * du.abs().max().item()
    assert torch.allclose(df, y.float().cpu(), rtol=0.3, atol=0.1 * y.float().abs().max().item())
    o_f = ops.linear(fused, down, out_f32=True)
    o_u = ops.linear(unfused, down, out_f32=True)
    _close(o_f, o_u, rtol=5e-2, atol=6e-2 * o_u.abs().max().item())   # a few flipped e2m1 codes over K = 10240
    # shapes the persistent kernel does not serve fall back to GEMM + row kernel, same result type
    small = ops.make_weight(ops.interleave_gate_up(wg[:256], wu[:256]), "nvfp4").to(DEV)
    fb = ops.linear(a, small, swiglu=True, quant_out=gs)
    assert fb.fmt == "nvfp4" and fb.K == 256
    ops.check_status(DEV)


@pytest.mark.parametrize("heads", [(40, 8), (5, 1)])
@pytest.mark.parametrize("ctx_lens,part_tokens", [([5, 130, 64, 700], 0), ([300, 1025], 256)])
def test_attention_epilogue_quantises_to_nvfp4_with_a_static_scale(ctx_lens, part_tokens, heads):
    """Decode attention writing packed e2m1 + tiled scale factors for o_proj (direct store and the
    last-arriver merge of several partitions) against the row kernel applied to its bf16 output.
    (5, 1) is one rank's share under 8-way tensor parallelism: 640 channels do not fill a
    256-channel scale-factor stage, so the padding groups come from a pre-zeroed buffer."""
    fp8, D = True, 128
    Hq, Hkv = heads
    q_lens = [1] * len(ctx_lens)
    args, want = _attn_case(fp8, D, Hq, Hkv, q_lens, ctx_lens, build_only=True)
    o = ops.paged_attention(*args["pos"], **args["kw"], part_tokens=part_tokens)
    gs = float(o.float().abs().max()) * 1.5 / (6 * 448)
    fused = ops.paged_attention(*args["pos"], **args["kw"], part_tokens=part_tokens, quant_out=gs)
    unfused = ops.quantize_act(o.view(o.shape[0], Hq * D), "nvfp4", static_scale=gs)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert fused.fmt == "nvfp4" and fused.K == Hq * D
    df, du = _dequant_act(fused), _dequant_act(unfused)
    assert (df == du).float().mean().item() > 0.97
    assert torch.allclose(df, o.float().cpu().view(len(q_lens), -1), rtol=0.3, atol=0.1 * o.float().abs().max().item())


def test_sf_repack_matches_reference_layout():
    sf = torch.randint(0, 120, (300, 40), dtype=torch.uint8)
    w = ops.QuantWeight("nvfp4", 300, 640, torch.zeros(300, 320, dtype=torch.uint8), sf, 1.0).to(DEV)
    want = ref.sf_to_tiled(sf, w.sf_k64).flatten()
    assert torch.equal(w.sf_tiled.cpu(), want)


@pytest.mark.parametrize("fmt", ["bf16", "fp8_row", "fp8_g128", "nvfp4"])
@pytest.mark.parametrize("K,with_res", [(1024, True), (1024, False), (17408, False), (5120, False)])
def test_rowop_rmsnorm_quant(fmt, K, with_res):
    M = 37
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    r = torch.randn(M, K, generator=g).to(torch.bfloat16) if with_res else None
    w = (torch.randn(K, generator=g) * 0.1).to(torch.bfloat16)
    a_ref, res_ref = ops.row_op(x, fmt, ops.IN_RMSNORM, residual=r, write_residual=with_res, w=w,
                                plus_one=True, eps=1e-6, also_bf16=True)
    a, res = ops.row_op(x.to(DEV), fmt, ops.IN_RMSNORM, residual=None if r is None else r.to(DEV),
                        write_residual=with_res, w=w.to(DEV), plus_one=True, eps=1e-6, also_bf16=True)
    if with_res:
        assert torch.equal(res.cpu(), res_ref)
    _close(a.bf16, a_ref.bf16, rtol=1e-2, atol=1e-2)
    # decode the kernel's encoding and compare with the oracle's dequantised matrix
    if fmt == "bf16":
        deq = a.data.float().cpu()
    elif fmt == "fp8_row":
        deq = ref.from_e4m3(a.data.cpu()) * a.scale.cpu()[:, None]
    elif fmt == "fp8_g128":
        deq = ref.from_e4m3(a.data.cpu()) * a.scale.cpu()[:, :M].t().repeat_interleave(128, 1)[:, :K]
    else:
        sf = ref.tiled_to_sf(a.sf.cpu().view(-1, a.sf_k64, 512), M, K // 16)
        deq = ref.dequantize_nvfp4(a.data.cpu(), sf, a.scale.cpu())
    # quantisation bins can flip on 1-ulp differences of the normalised value: allow one step
    step = a_ref.data.abs().amax(dim=1, keepdim=True) * (0.3 if fmt == "nvfp4" else 0.08)
    assert ((deq - a_ref.data).abs() <= step + 1e-3).all()
    assert ((deq - a_ref.data).abs() > 1e-3).float().mean() < 0.02


def test_rowop_activations():
    M, K = 19, 512
    g = torch.Generator().manual_seed(4)
    x = torch.randn(M, 2 * K, generator=g).to(torch.bfloat16)
    for mode, kk in ((ops.IN_SILU_MUL, K), (ops.IN_RELU2, 2 * K)):
        want, _ = ops.row_op(x, "bf16", mode, K=kk)
        got, _ = ops.row_op(x.to(DEV), "bf16", mode, K=kk)
        _close(got.data, want.data, 1e-2, 1e-2)
    for fmt in ("nvfp4", "fp8_g128", "fp8_row"):
        want, _ = ops.row_op(x, fmt, ops.IN_SILU_MUL, K=K, also_bf16=True)
        got, _ = ops.row_op(x.to(DEV), fmt, ops.IN_SILU_MUL, K=K, also_bf16=True)
        _close(got.bf16, want.bf16, 1e-2, 1e-2)
        wfmt = {"nvfp4": "nvfp4", "fp8_g128": "fp8_block", "fp8_row": "fp8_row"}[fmt]
        got_lin = ops.linear(got, ops.make_weight(torch.eye(K)[:128], wfmt).to(DEV), out_f32=True)
        _close(got_lin, want.data[:, :128], 0.3, 0.3 * want.data.abs().max().item())
    # sigmoid gate interleaved per head: [Q_h | G_h] with head_dim 64
    H, D = 4, 64
    attn = torch.randn(M, H * D, generator=g).to(torch.bfloat16)
    qg = torch.randn(M, H * 2 * D + 100, generator=g).to(torch.bfloat16)
    kw = dict(gate=qg, head_dim=D, gate_head_stride=2 * D, gate_head_off=D)
    want, _ = ops.row_op(attn, "bf16", ops.IN_SIGMOID_GATE, **kw)
    kw["gate"] = qg.to(DEV)
    got, _ = ops.row_op(attn.to(DEV), "bf16", ops.IN_SIGMOID_GATE, **kw)
    _close(got.data, want.data, 1e-2, 1e-2)
    # gated rmsnorm over groups with an fp32 input
    xf = torch.randn(M, K, generator=g)
    z = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(128, generator=g).abs().to(torch.bfloat16).repeat(K // 128)
    want, _ = ops.row_op(xf, "bf16", ops.IN_GATED_RMSNORM, gate=z, w=w, group=128)
    got, _ = ops.row_op(xf.to(DEV), "bf16", ops.IN_GATED_RMSNORM, gate=z.to(DEV), w=w.to(DEV), group=128)
    _close(got.data, want.data, 1e-2, 1e-2)


def test_kv_write_observes_amax_and_rescale_matches_reference():
    """Online FP8 KV calibration support: the KV-write kernel accumulates max |k| / max |v| of the
    rows it writes, and kv_rescale re-encodes the listed slots from one scale to another."""
    M, Hq, Hkv, D, bs, nb = 19, 4, 2, 128, 16, 6
    g = torch.Generator().manual_seed(8)
    qkv = (torch.randn(M, (Hq + 2 * Hkv) * D, generator=g) * 3).to(torch.bfloat16)
    pos = torch.arange(M, dtype=torch.int32)
    slots = torch.randperm(nb * bs, generator=g)[:M].to(torch.int64)
    slots[5] = -1
    cos, sin = ref.rope_tables(64, D, 1e6)
    two = torch.tensor([2.0])
    kc, vc = _cache(nb, bs, Hkv, D, True)
    am_ref = torch.zeros(2)
    ops.qk_norm_rope_kvwrite(qkv, Hq=Hq, Hkv=Hkv, D=D, positions=pos, slots=slots, k_cache=kc, v_cache=vc, cos=cos, sin=sin,
                             k_scale=two, v_scale=two, amax=am_ref)
    kcg, vcg = kc.clone().zero_().to(DEV), vc.clone().zero_().to(DEV)
    am = torch.zeros(2, device=DEV)
    ops.qk_norm_rope_kvwrite(qkv.to(DEV), Hq=Hq, Hkv=Hkv, D=D, positions=pos.to(DEV), slots=slots.to(DEV), k_cache=kcg,
                             v_cache=vcg, cos=cos.to(DEV), sin=sin.to(DEV), k_scale=two.to(DEV), v_scale=two.to(DEV), amax=am)
    torch.cuda.synchronize()
    assert (am.cpu() - am_ref).abs().max() <= 2e-2 * am_ref.max()
    new = (am.cpu()[:1] / 448).clone()
    want = kc.clone()
    ops.kv_rescale(want, slots, 2.0, new)
    ops.kv_rescale(kcg, slots.to(DEV), 2.0, new.to(DEV))
    torch.cuda.synchronize()
    ops.check_status(DEV)
    a, b = ref.from_e4m3(kcg.cpu()), ref.from_e4m3(want)
    assert ((a - b).abs() <= 0.13 * b.abs() + 1e-6).all() and (kcg.cpu() != want).float().mean() < 0.02
    live = slots[slots >= 0]
    assert ref.from_e4m3(want).view(nb * bs, -1)[live].abs().max() > 200        # the rows now use the e4m3 range


def _cache(nb, bs, Hkv, D, fp8):
    dt = torch.uint8 if fp8 else torch.bfloat16
    return torch.zeros(nb, bs, Hkv, D, dtype=dt), torch.zeros(nb, bs, Hkv, D, dtype=dt)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("q_lens,ctx_lens", [([128], [128]), ([200, 130], [200, 391]), ([384, 5, 131], [384, 70, 400]),
                                             ([1024], [1024])])
def test_prefill_attention_on_tcgen05_matches_fp32_oracle(fp8, q_lens, ctx_lens):
    """Both products of a 128-row query tile as tcgen05.mma with TMEM accumulators
    (csrc/attention_tc.cu): fresh prefills, chunks that continue a cached prefix, ragged tails,
    short sequences in the same launch, GQA (8 query heads per 2 KV heads), bf16 and e4m3 caches."""
    _attn_case(fp8, 128, 8, 2, q_lens, ctx_lens, force_mode=3)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("q_lens,ctx_lens", [([200, 130], [200, 391]), ([512], [512])])
def test_prefill_attention_on_tcgen05_head_dim_256(fp8, q_lens, ctx_lens):
    """The same kernel at head_dim 256 (four 64-dim blocks per row, O in 256 TMEM columns, V read
    as an MN-major operand): the attention layers of the Qwen3-Next style hybrids."""
    _attn_case(fp8, 256, 4, 2, q_lens, ctx_lens, force_mode=3)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("D,rot", [(128, 128), (64, 64), (256, 64), (64, 32), (128, 32)])
def test_rope_kvwrite(fp8, D, rot):
    M, Hq, Hkv, bs, nb = 23, 8, 2, 16, 12
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(M, (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 500, (M,), generator=g, dtype=torch.int32)
    slots = torch.randperm(nb * bs, generator=g)[:M].to(torch.int64)
    slots[3] = -1
    qn = (torch.randn(D, generator=g) * 0.1).to(torch.bfloat16)
    kn = (torch.randn(D, generator=g) * 0.1).to(torch.bfloat16)
    cos, sin = ref.rope_tables(512, rot, 1e6)
    ks, vs = torch.tensor([0.02]), torch.tensor([0.015])
    kc, vc = _cache(nb, bs, Hkv, D, fp8)
    q_ref = ops.qk_norm_rope_kvwrite(qkv, Hq=Hq, Hkv=Hkv, D=D, positions=pos, slots=slots, k_cache=kc,
                                     v_cache=vc, q_norm_w=qn, k_norm_w=kn, plus_one=True, cos=cos,
                                     sin=sin, k_scale=ks, v_scale=vs)
    kcg, vcg = kc.clone().zero_().to(DEV), vc.clone().zero_().to(DEV)
    q = ops.qk_norm_rope_kvwrite(qkv.to(DEV), Hq=Hq, Hkv=Hkv, D=D, positions=pos.to(DEV),
                                 slots=slots.to(DEV), k_cache=kcg, v_cache=vcg, q_norm_w=qn.to(DEV),
                                 k_norm_w=kn.to(DEV), plus_one=True, cos=cos.to(DEV), sin=sin.to(DEV),
                                 k_scale=ks.to(DEV), v_scale=vs.to(DEV))
    _close(q, q_ref, 2e-2, 2e-2)
    if fp8:
        _close(ref.from_e4m3(kcg.cpu()), ref.from_e4m3(kc), 0.13, 1.0)   # one e4m3 step
        assert (kcg.cpu() != kc).float().mean() < 0.02
        _close(ref.from_e4m3(vcg.cpu()), ref.from_e4m3(vc), 0.13, 1.0)
        assert (vcg.cpu() != vc).float().mean() < 0.02
    else:
        _close(kcg, kc, 2e-2, 2e-2)
        assert torch.equal(vcg.cpu(), vc)
    ops.check_status(DEV)


def _attn_case(fp8, D, Hq, Hkv, q_lens, ctx_lens, window=0, force_mode=0, seed=6, build_only=False):
    bs = 16
    g = torch.Generator().manual_seed(seed)
    S = len(q_lens)
    max_blocks = (max(ctx_lens) + bs - 1) // bs
    nb = S * max_blocks + 3
    perm = torch.randperm(nb, generator=g)
    bt = torch.full((S, max_blocks), -1, dtype=torch.int32)
    used = 0
    for s in range(S):
        n = (ctx_lens[s] + bs - 1) // bs
        bt[s, :n] = perm[used:used + n].to(torch.int32)
        used += n
    if fp8:
        kc = torch.randint(0, 256, (nb, bs, Hkv, D), generator=g, dtype=torch.uint8)
        vc = torch.randint(0, 256, (nb, bs, Hkv, D), generator=g, dtype=torch.uint8)
        kc[(kc & 0x7F) == 0x7F] = 0x30   # no NaN codes
        vc[(vc & 0x7F) == 0x7F] = 0x30
        kc = (kc & 0xBF) | 0x20          # keep magnitudes moderate
        vc = (vc & 0xBF) | 0x20
        ks, vs = torch.tensor([0.05]), torch.tensor([0.03])
    else:
        kc = torch.randn(nb, bs, Hkv, D, generator=g).to(torch.bfloat16)
        vc = torch.randn(nb, bs, Hkv, D, generator=g).to(torch.bfloat16)
        ks = vs = None
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    q_len = torch.tensor(q_lens, dtype=torch.int32)
    q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
    ctx = torch.tensor(ctx_lens, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    want = ref.paged_attention(q, kc, vc, bt.clamp(min=0), q_start, q_len, ctx, scale, ks, vs, window)
    dv = lambda t: None if t is None else t.to(DEV)
    if build_only:
        return dict(pos=(dv(q), dv(kc), dv(vc), dv(bt.clamp(min=0)), dv(q_start), dv(q_len), dv(ctx)),
                    kw=dict(max_q_len=max(q_lens), max_ctx=max(ctx_lens), scale=scale, k_scale=dv(ks), v_scale=dv(vs),
                            window=window, force_mode=force_mode)), want
    got = ops.paged_attention(dv(q), dv(kc), dv(vc), dv(bt.clamp(min=0)), dv(q_start), dv(q_len), dv(ctx),
                              max_q_len=max(q_lens), max_ctx=max(ctx_lens), scale=scale, k_scale=dv(ks),
                              v_scale=dv(vs), window=window, force_mode=force_mode)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    _close(got, want, 2e-2, 2e-2 * max(1.0, want.abs().max().item()))


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_decode_gqa5_d128(fp8):
    _attn_case(fp8, 128, 40, 8, [1, 1, 1, 1], [1, 17, 640, 1153])


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_verify_rows(fp8):
    _attn_case(fp8, 128, 40, 8, [5, 5, 3], [133, 700, 64])       # 25 rows: two m16 tiles
    _attn_case(fp8, 64, 4, 2, [1, 4, 2], [33, 100, 2])


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_decode_d256(fp8):
    _attn_case(fp8, 256, 16, 2, [1, 1], [90, 600])
    _attn_case(fp8, 256, 16, 2, [4, 1], [90, 600])                # falls back to row-wise sequences


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("D", [64, 128, 256])
def test_attention_prefill(fp8, D):
    Hq, Hkv = (8, 2) if D != 64 else (4, 2)
    _attn_case(fp8, D, Hq, Hkv, [128, 70, 200], [128, 170, 200])   # fresh, chunked-after-cache, fresh


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_short_verify_chunks_on_the_prefill_path(fp8):
    """Verify steps with more than 32 query rows per KV head group (8 drafts + 1, GQA 4) take the
    split-Q kernel with short, ragged chunks that start deep inside the context, also mixed
    with single-row sequences."""
    _attn_case(fp8, 128, 8, 2, [9, 9], [28, 25])
    _attn_case(fp8, 128, 8, 2, [9, 1], [28, 30])
    _attn_case(fp8, 128, 8, 2, [1, 9, 2], [40, 21, 77])
    _attn_case(fp8, 128, 8, 2, [9, 9, 9, 5], [200, 9, 130, 64])


def test_attention_sliding_window():
    _attn_case(False, 128, 8, 2, [1, 1], [300, 900], window=128)
    _attn_case(False, 128, 8, 2, [100], [400], window=64)


def test_argmax_and_logprob():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(9, 151936, generator=g).to(torch.bfloat16)
    x[2, 5] = x[2, 77] = 50.0                                       # tie -> lower index
    ids_ref, lp_ref = ops.argmax(x, logprob=True, mask_ids=(3, -1))
    ids, lp = ops.argmax(x.to(DEV), logprob=True, mask_ids=(3, -1))
    assert torch.equal(ids.cpu(), ids_ref)
    _close(lp, lp_ref, 1e-3, 1e-3)
    xf = torch.randn(4, 4096, generator=g)
    assert torch.equal(ops.argmax(xf.to(DEV)).cpu(), ops.argmax(xf))
    # bf16 rows read with 16-byte loads: ragged tail (V % 8 != 0), maxima in the last lanes and in
    # the tail, negative-only rows, a masked maximum, an odd row pitch (the scalar path)
    xb = (torch.randn(6, 1003, generator=g) - 4.0).to(torch.bfloat16)
    xb[0, 1002] = 9.0
    xb[1, 999] = 9.0
    xb[2, 7] = xb[2, 8] = 9.0
    xb[3, 500] = 9.0
    assert torch.equal(ops.argmax(xb.to(DEV)).cpu(), ops.argmax(xb))
    assert torch.equal(ops.argmax(xb.to(DEV), mask_ids=(500, 1002)).cpu(), ops.argmax(xb, mask_ids=(500, 1002)))
    wide = torch.randn(5, 1024, generator=g).to(torch.bfloat16)
    assert torch.equal(ops.argmax(wide.to(DEV)).cpu(), ops.argmax(wide))


def test_sample_matches_reference_draws():
    g = torch.Generator().manual_seed(8)
    M, V = 12, 4096
    x = torch.randn(M, V, generator=g) * 3
    temp = torch.tensor([0.0, 1.0, 0.7, 1.3] * 3)
    top_k = torch.tensor([0, 0, 50, 5] * 3, dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.8] * 3)
    min_p = torch.tensor([0.0, 0.0, 0.05, 0.0] * 3)
    seed = torch.arange(M, dtype=torch.int64) + 42
    step = torch.arange(M, dtype=torch.int64)
    ids_ref, lp_ref = ops.sample(x, temp, top_k, top_p, min_p, seed, step)
    d = lambda t: t.to(DEV)
    ids, lp = ops.sample(d(x), d(temp), d(top_k), d(top_p), d(min_p), d(seed), d(step))
    ids = ids.cpu()
    # every draw must land inside the reference keep-set; exact equality except when the
    # uniform draw falls within float noise of a cumulative boundary
    for r in range(M):
        if temp[r] <= 0:
            assert ids[r] == ids_ref[r]
        else:
            keep = ops.sample_keep_mask(x[r], float(temp[r]), int(top_k[r]), float(top_p[r]), float(min_p[r]))
            assert keep[ids[r]]
    assert (ids == ids_ref).float().mean() >= 0.75
    same = ids == ids_ref
    _close(lp.cpu()[same], lp_ref[same], 1e-3, 1e-3)


def test_embed_and_bounds_status():
    table = torch.randn(100, 64).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([0, 99, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embed(ids, table), table[ids.long()])
    bad = torch.tensor([0, 100], dtype=torch.int32, device=DEV)
    out = ops.embed(bad, table)
    assert out[1].abs().sum() == 0
    with pytest.raises(Exception):
        ops.check_status(DEV)
    assert ops.check_status(DEV) == 0
