"""Roofline planner and signed benchmark gate records (pure host logic)."""
import json

import pytest

from metrale_inference_alpha_b200.bench.gate import GateRecord, kernel_closure_hash, new_signing_key
from metrale_inference_alpha_b200.config.model_config import preset
from metrale_inference_alpha_b200.planner import DevicePeaks, decode_step_ops, estimate


def test_planner_bytes_match_the_model_and_scale_with_batch_and_tp():
    cfg = preset("dense-27b-nvfp4")
    peaks = DevicePeaks(hbm_gbs=6449.1, bf16_tflops=1388.9)
    e1, e128 = estimate(cfg, 1, 640, peaks=peaks), estimate(cfg, 128, 640, peaks=peaks)
    # weights: ~27B params at 0.5625 B + bf16 lm_head; the decode step streams them once
    assert 13.0 < e1["gbytes_per_step"] < 14.5
    assert e128["gbytes_per_step"] - e1["gbytes_per_step"] > 10.0          # KV stream of 128 sequences
    assert e1["step_ms_bytes_only"] == pytest.approx(e1["gbytes_per_step"] / 6449.1 * 1e3, rel=1e-3)
    assert e128["step_ms_roofline_per_op"] >= e128["step_ms_bytes_only"]
    attn = next(r for r in e128["ops"] if r["op"] == "paged attention")
    assert attn["bound"] == "memory" and 165 < attn["mbytes_each"] < 175    # 128 x 640 x 8 x 128 x 2 bytes
    tp8 = estimate(cfg, 128, 640, tp=8, peaks=peaks)
    assert tp8["gbytes_per_step"] < e128["gbytes_per_step"] / 4
    assert e1["launches"] == e128["launches"] and 500 < e1["launches"] < 530
    names = [o.name for o in decode_step_ops(preset("qwen-hybrid-moe-35b-fp8"), 16, 640)]
    assert "moe experts" in names and "recurrent state update" in names
    assert any(o.name == "mla attention" for o in decode_step_ops(preset("deepseek-v3-671b-fp8"), 16, 640, tp=8))


def test_cli_plan_prints_a_table(capsys):
    from metrale_inference_alpha_b200.server import cli
    assert cli.main(["plan", "--model", "dense-27b-nvfp4", "--batch", "16", "--json"]) == 0
    d = json.loads(capsys.readouterr().out)
    assert d["batch"] == 16 and d["ops"]


def test_gate_record_signing_tamper_detection_and_regression(tmp_path):
    line = {"metric": "aggregate decode tok/s", "value": 13685.0, "unit": "tokens/s", "higher_is_better": True,
            "config": {"model": "dense-27b-nvfp4", "global_batch": 128}}
    key = new_signing_key()
    rec = GateRecord.from_bench_line("c128", line, device="B200").sign(key)
    assert rec.closure == kernel_closure_hash() and len(rec.closure) == 64
    assert rec.verify() and rec.verify(rec.public_key) and not rec.verify("AAAA")
    rec.save(tmp_path / "r.json")
    back = GateRecord.load(tmp_path / "r.json")
    assert back.verify() and back.digest() == rec.digest()
    back.value = 99999.0
    assert not back.verify()                                   # edited after signing
    assert rec.passes(13000.0) and not rec.passes(14000.0)
    slower = GateRecord("c128", rec.metric, 12000.0, rec.unit)
    assert "0.877x" in slower.regression_vs(rec)
    assert GateRecord("c128", rec.metric, 13500.0, rec.unit).regression_vs(rec) is None
    assert "not comparable" in GateRecord("x", "ttft", 1.0, "ms", False).regression_vs(rec)


def test_recipe_yaml_to_serve_arguments(tmp_path):
    from metrale_inference_alpha_b200.config.recipes import load_recipe, recipe_to_argv
    from metrale_inference_alpha_b200.server import cli
    p = tmp_path / "r.yaml"
    p.write_text("model: tiny-dense\nmax-num-seqs: 16\nuse_cuda_graphs: false\ntool_call_parser: mistral\n"
                 "lora_adapters: {sql: /a/sql}\napi_key: [k1, k2]\nenv: {METRALE_PDL: '0'}\n")
    argv = cli._apply_recipe(["serve", "--recipe", str(p), "--port", "9001", "--max-num-seqs", "4"])
    ns = cli.build_parser().parse_args(argv)
    assert ns.model == "tiny-dense" and ns.max_num_seqs == 4 and ns.port == 9001        # command line wins
    assert ns.use_cuda_graphs is False and ns.tool_call_parser == "mistral"
    assert ns.lora_adapter == ["sql=/a/sql"] and ns.api_key == ["k1", "k2"]
    p.write_text("model: x\nnot_an_option: 1\n")
    with pytest.raises(ValueError, match="not a serve option"):
        recipe_to_argv(load_recipe(str(p)), ["--model"])
    p.write_text("model: x\nenv: {METRALE_TYPO: 1}\n")
    with pytest.raises(ValueError, match="undeclared levers"):
        recipe_to_argv(load_recipe(str(p)), ["--model"])


def test_launch_trace_records_and_diffs():
    from metrale_inference_alpha_b200.ops import _native
    with _native.launch_trace() as a:
        _native.check(0, "gemm[nvfp4 M=1 N=2 K=3]")
        _native.check(0, "row_op")
    with _native.launch_trace() as b:
        _native.check(0, "gemm[bf16 M=9]")
        _native.check(0, "paged_attention")
    assert a == ["gemm", "row_op"] and _native.diff_traces(a, b) == (1, "row_op", "paged_attention")
    assert _native.diff_traces(a, a) is None and _native.diff_traces(a, a[:1]) == (1, "row_op", None)
    _native.check(0, "not recorded")
