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
