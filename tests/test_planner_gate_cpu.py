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


# ----------------------------------------------------------------------------- OTLP export
def test_otlp_body_and_push_to_a_local_collector():
    import http.server
    import json as _json
    import threading

    from metrale_inference_alpha_b200.utils.otlp import OtlpExporter, metrics_body
    from metrale_inference_alpha_b200.utils.telemetry import Telemetry
    tel = Telemetry("basic")
    tel.inc("decode_tokens", 41)
    tel.inc("decode_tokens")
    tel.inc("energy_joules", 0.5)
    tel.set("kv_blocks_free", 17)
    for ms in (0.5, 3, 3, 40000):
        tel.observe_ms("step", ms)
    body = metrics_body(tel, {"running": 2, "name": "skip-me"}, now_ns=123)
    ms = {m["name"]: m for m in body["resourceMetrics"][0]["scopeMetrics"][0]["metrics"]}
    assert ms["metrale.decode_tokens"]["sum"]["dataPoints"][0]["asInt"] == "42"
    assert ms["metrale.decode_tokens"]["sum"]["isMonotonic"] and ms["metrale.decode_tokens"]["unit"] == "{token}"
    assert ms["metrale.energy_joules"]["sum"]["dataPoints"][0]["asDouble"] == 0.5
    assert ms["metrale.kv_blocks_free"]["gauge"]["dataPoints"][0]["asDouble"] == 17.0
    assert ms["metrale.running"]["gauge"]["dataPoints"][0]["timeUnixNano"] == "123" and "metrale.name" not in ms
    h = ms["metrale.step"]["histogram"]["dataPoints"][0]
    assert h["count"] == "4" and len(h["bucketCounts"]) == len(h["explicitBounds"]) + 1
    assert h["bucketCounts"][0] == "1" and h["bucketCounts"][-1] == "1" and abs(h["sum"] - 40006.5) < 1e-6

    got = []

    class H(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            got.append((self.path, _json.loads(self.rfile.read(int(self.headers["Content-Length"])))))
            self.send_response(200)
            self.end_headers()

        def log_message(self, *a):
            pass
    srv = http.server.HTTPServer(("127.0.0.1", 0), H)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    try:
        ex = OtlpExporter(tel, f"http://127.0.0.1:{srv.server_port}", period_s=0.05).start()
        import time as _t
        end = _t.time() + 5
        while not got and _t.time() < end:
            _t.sleep(0.02)
        ex.stop()
        assert got and got[0][0] == "/v1/metrics" and ex.pushed >= 2 and ex.failed == 0
        assert got[-1][1]["resourceMetrics"][0]["resource"]["attributes"][0]["value"]["stringValue"] == "metrale-b200"
    finally:
        srv.shutdown()
    dead = OtlpExporter(tel, "http://127.0.0.1:9", period_s=60)
    assert dead.export_once() is False and dead.failed == 1          # a dead collector never raises


# ----------------------------------------------------------------------------- change ledger
def test_ledger_journey_dedup_graph_and_mergeability(tmp_path):
    from metrale_inference_alpha_b200.bench import ledger as L
    p = L.path_for(tmp_path, 42)
    ev = [
        L.Event.state(42, "aaa", "open", at=1),
        L.Event.gate(42, "aaa", "unit-tests", "pass", run_id="r1", at=2),
        L.Event.gate(42, "aaa", "bench-gate", "fail", invalidated_by=["kernel-closure"], detail="-7% tok/s", run_id="r1", at=3),
        L.Event.gate(42, "aaa", "unit-tests", "pass", run_id="r1", at=2),           # CI retry replays the line
        L.Event.measurement(42, "bbb", "decode_c128", {"tok_s": 14240.0, "ttft_ms": 506.0}, run_id="r2", at=5),
        L.Event.gate(42, "bbb", "unit-tests", "pass", run_id="r2", at=6),
        L.Event.gate(42, "bbb", "bench-gate", "pass", invalidated_by=["kernel-closure"], run_id="r2", at=7),
        L.Event.category(42, "bbb", "perf", "confirmed", at=8),
    ]
    for e in ev:
        L.append(p, e)
    j = L.read_all(p)
    assert len(j.events) == 8 and j.events[4].payload["metrics"]["tok_s"] == 14240.0
    assert L.Event.from_json(ev[2].to_json()).identity() == ev[2].identity()
    d = j.deduplicated()
    assert len(d.events) == 7
    assert [e.payload["verdict"] for e in d.gate_history("bench-gate")] == ["fail", "pass"]
    ok, why = d.mergeable(["unit-tests", "bench-gate"])
    assert ok and not why
    ok, why = d.mergeable(["unit-tests", "bench-gate", "signed-record"])
    assert not ok and "signed-record" in why[0]
    # a later kernel-closure event invalidates the bench gate that named it
    L.append(p, L.Event.gate(42, "bbb", "kernel-closure", "pass", run_id="r3", at=9))
    ok, why = L.read_all(p).deduplicated().mergeable(["unit-tests", "bench-gate"])
    assert not ok and "invalidated" in why[0]
    g = L.materialize(d)
    commits = [n for n in g.nodes if n["label"] == "commit"]
    assert [c["sha"] for c in commits] == ["aaa", "bbb"]
    assert len(g.out(0, "observed")) == 3 and len(g.out(1, "observed")) == 4
    assert sum(1 for e in g.edges if e[2] == "precedes") == 6
    with pytest.raises(ValueError):
        L.Event.gate(1, "x", "g", "maybe")
    p.write_text(p.read_text() + "{not json\n")
    with pytest.raises(ValueError, match="line"):
        L.read_all(p)


def test_nvtx_ranges_are_noops_without_cuda(monkeypatch):
    from metrale_inference_alpha_b200.utils import nvtx
    monkeypatch.setattr(nvtx, "_enabled", None)
    monkeypatch.setenv("METRALE_NVTX", "1")
    with nvtx.range("x"):
        nvtx.mark("y")
    import torch
    assert nvtx.enabled() == torch.cuda.is_available()
    monkeypatch.setattr(nvtx, "_enabled", None)
