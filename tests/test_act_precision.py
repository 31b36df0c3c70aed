"""Activation precision options of the quantised linears.

(1) W4A16 / W8A16: bf16 activations against NVFP4 / FP8 weights (ops/csrc/a16.cu), compared
    with the fp32 reference ``x @ dequant(W)^T`` for the streaming kernel (M <= 32) and the
    widen-then-tensor-core path (larger M), with the residual and SwiGLU epilogues.
(2) Static against dynamic NVFP4 activation scales on rows with outliers: the evidence behind the
    engine's defaults (a calibrated scale with a 2x margin for the epilogue-fused quantisers;
    "a16" for checkpoints whose activations leave the calibrated range). Same quantisation rule as
    the reference's NVFP4 quantiser (kernels/gb10/common/quantize_bf16_to_nvfp4.cu:2-16).
"""
import pytest
import torch

from metrale_inference_alpha_b200 import ops
from metrale_inference_alpha_b200.ops import reference as ref


def _weights(fmt, N, K, g):
    return ops.make_weight(torch.randn(N, K, generator=g) * 0.05, fmt)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "fp8_row", "fp8_block"])
@pytest.mark.parametrize("M", [1, 3, 8, 20, 200])
def test_a16_linear_matches_fp32_reference(fmt, M):
    g = torch.Generator().manual_seed(M)
    N, K = 1280, 2304
    w = _weights(fmt, N, K, g)
    x = (torch.randn(M, K, generator=g)).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    want = x.float() @ w.dequant().t()
    wd = w.to("cuda")
    act = ops.Act("bf16", M, K, x.cuda())
    got = ops.linear(act, wd, out_f32=True).cpu()
    tol = 2e-2 if M > 32 else 2e-3                     # the tensor-core path rounds the widened weight to bf16
    assert (got - want).abs().max() <= tol * want.abs().max()
    got_r = ops.linear(act, wd, residual=res.cuda()).float().cpu()
    want_r = want + res.float()
    assert (got_r - want_r).abs().max() <= 2e-2 * want_r.abs().max()
    got_s = ops.linear(act, wd, swiglu=True, out_f32=True).cpu()
    want_s = torch.nn.functional.silu(want[:, 0::2]) * want[:, 1::2]
    assert (got_s - want_s).abs().max() <= max(tol, 5e-3) * want_s.abs().max() + 1e-4
    torch.cuda.synchronize()
    ops.check_status("cuda")


def test_activation_precision_switch_and_engine_runs_a16_on_cpu():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    try:
        eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=2, max_model_len=128,
                                   activation_precision="a16"))
        assert set(ops.ACT_FOR_WEIGHT.values()) == {"bf16"}
        out = eng.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=6))[0].output_ids
        assert len(out) == 6
    finally:
        ops.set_activation_precision("native")
    assert ops.ACT_FOR_WEIGHT == ops.NATIVE_ACT_FOR_WEIGHT


def _rel_err(a, b):
    return float((a - b).norm() / b.norm())


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
def test_static_against_dynamic_nvfp4_activation_scales_on_outlier_rows(device):
    """Three row populations through the same NVFP4 GEMM, as relative error of the product:
    typical rows (inside the calibration range), small rows (1/256 of it) and outlier rows
    (8x the calibration maximum). Findings the defaults rest on:
      * inside the calibrated range the static scale costs nothing measurable (the e4m3 block
        scales absorb the difference): <= 1.1x the dynamic error, also for small rows;
      * beyond margin x calibrated amax the static quantiser clips (error 2.5x the
        dynamic one), while bf16 activations ("a16") are exact to rounding everywhere.
    So: static scales (margin 2) where the quantiser is fused into a GEMM epilogue, dynamic
    per-row scales everywhere else, and a16 as the accuracy option."""
    g = torch.Generator().manual_seed(3)
    M, K, N = 96, 2048, 512
    w = _weights("nvfp4", N, K, g)
    typical = torch.randn(M, K, generator=g)
    typical[:, ::97] *= 6.0                                  # a few strong channels, as in SwiGLU outputs
    calib_amax = float(typical.abs().max())
    static = 2.0 * calib_amax / (6.0 * 448.0)
    rows = {"typical": typical, "small": typical / 256.0, "outlier": typical * 8.0}
    wq = w.to(device) if device == "cuda" else w
    err = {}
    for name, x in rows.items():
        exact = x @ w.dequant().t()
        xb = x.to(torch.bfloat16)
        for mode, scale in (("dynamic", 0.0), ("static", static)):
            if device == "cuda":
                a = ops.quantize_act(xb.cuda(), "nvfp4", static_scale=scale)
                y = ops.linear(a, wq, out_f32=True).cpu()
            else:
                y = ops.encode_act_ref(xb.float(), "nvfp4", static_scale=scale).data @ w.dequant().t()
            err[name, mode] = _rel_err(y, exact)
        if device == "cuda":
            y16 = ops.linear(ops.Act("bf16", M, K, xb.cuda()), wq, out_f32=True).cpu()
        else:
            y16 = xb.float() @ w.dequant().t()
        err[name, "a16"] = _rel_err(y16, exact)
    for name in ("typical", "small"):
        assert err[name, "static"] <= 1.1 * err[name, "dynamic"] + 1e-4, err
    assert err["outlier", "static"] > 2.0 * err["outlier", "dynamic"], err      # 0.24 against 0.09 here
    for name in rows:
        assert err[name, "a16"] < 0.1 * err[name, "dynamic"], err
        assert err[name, "dynamic"] < 0.15, err
