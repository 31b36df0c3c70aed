"""Benchmark suites: function calling (draw, checker, aggregation, run through the HTTP app), the agentic
tool loop on a virtual workspace, request isolation and scheduler equivalence."""
import json

import pytest
import torch

from metrale_inference_alpha_b200.bench import agentic as AG
from metrale_inference_alpha_b200.bench import function_calling as FC
from metrale_inference_alpha_b200.bench.isolation import contamination, scheduler_equivalence
from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine


def _call(name, **args):
    return {"tool_calls": [{"id": "c1", "type": "function", "function": {"name": name, "arguments": json.dumps(args)}}]}


def test_checker_accepts_equivalent_values_and_names_the_first_mismatch():
    s = {x.id: x for x in FC.load_dataset()}
    ok = FC.check_sample(s["simple_0"], FC.calls_of_message(_call("get_weather", city=" paris ", unit="celsius")))
    assert ok.ok
    assert FC.check_sample(s["simple_0"], FC.calls_of_message(_call("get_weather", city="Paris"))).ok        # optional unit
    assert FC.check_sample(s["simple_1"], FC.calls_of_message(_call("triangle_area", base=10.0, height=5))).ok
    assert not FC.check_sample(s["simple_1"], FC.calls_of_message(_call("triangle_area", base=10.0, height="5"))).ok     # a string is not a number
    bad = FC.check_sample(s["simple_0"], FC.calls_of_message(_call("get_weather", city="Lyon")))
    assert not bad.ok and "city" in bad.reason
    assert "unexpected" in FC.check_sample(s["simple_0"], FC.calls_of_message(_call("get_weather", city="Paris", day=1))).reason
    assert "missing" in FC.check_sample(s["simple_1"], FC.calls_of_message(_call("triangle_area", base=10))).reason
    assert "expected" in FC.check_sample(s["multiple_0"], FC.calls_of_message(_call("get_stock_price", symbol="X"))).reason
    # parallel: order-free, each expected call claims its own produced call
    two = {"tool_calls": _call("get_weather", city="Oslo")["tool_calls"] + _call("get_weather", city="Rome")["tool_calls"]}
    assert FC.check_sample(s["parallel_0"], FC.calls_of_message(two)).ok
    dup = {"tool_calls": _call("get_weather", city="Oslo")["tool_calls"] * 2}
    assert not FC.check_sample(s["parallel_0"], FC.calls_of_message(dup)).ok
    assert FC.check_sample(s["irrelevance_0"], []).ok and not FC.check_sample(s["irrelevance_0"], FC.calls_of_message(_call("get_weather", city="x"))).ok


def test_draw_is_deterministic_stratified_and_shards_partition(tmp_path):
    rows = [dict(FC.SMOKE_SET[i % 5], id=f"{FC.SMOKE_SET[i % 5]['category']}_{i}") for i in range(40)]
    p = tmp_path / "d.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    data = FC.load_dataset(str(p))
    a, b = FC.draw(data, 20, seed=3), FC.draw(data, 20, seed=3)
    assert [s.id for s in a] == [s.id for s in b] and len(a) == 20
    assert [s.id for s in FC.draw(data, 20, seed=4)] != [s.id for s in a]
    cats = {}
    for s in a:
        cats[s.category] = cats.get(s.category, 0) + 1
    assert cats == {"simple": 8, "multiple": 4, "parallel": 4, "irrelevance": 4}       # half of every category
    shards = [FC.draw(data, None, seed=1, shard=i, shards=3) for i in range(3)]
    ids = sorted(s.id for sh in shards for s in sh)
    assert ids == sorted(s.id for s in data)
    with pytest.raises(ValueError):
        FC.draw(data, 5, shard=3, shards=3)
    with pytest.raises(ValueError):
        p.write_text('{"id": "x"}')
        FC.load_dataset(str(p))


def test_run_and_aggregate_with_a_scripted_model():
    answers = {"simple_0": _call("get_weather", city="Paris"), "simple_1": _call("triangle_area", base=10, height=6),
               "multiple_0": _call("convert_currency", **{"amount": 100, "from": "usd", "to": "eur"}), "irrelevance_0": {"content": "why did..."}}
    data = FC.load_dataset()
    by_q = {s.question[0]["content"]: s.id for s in data}

    def ask(messages, tools):
        sid = by_q[messages[-1]["content"]]
        if sid == "parallel_0":
            raise RuntimeError("boom")
        assert tools and tools[0]["type"] == "function"
        return answers[sid]
    seen = []
    agg = FC.aggregate(FC.run(data, ask, on_progress=lambda i, n: seen.append((i, n))))
    assert seen[-1] == (5, 5) and agg["n"] == 5 and agg["correct"] == 3
    assert agg["categories"]["simple"] == {"n": 2, "correct": 1, "accuracy": 0.5} and agg["categories"]["parallel"]["correct"] == 0
    assert any("request failed" in f["reason"] for f in agg["failures"]) and "3 / 5" in FC.report(agg)
    assert len(FC.run(data, ask, should_stop=lambda: True)) == 0


def test_function_calling_through_the_http_app():
    from fastapi.testclient import TestClient
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    from metrale_inference_alpha_b200.server.tokenizer import load_tokenizer
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=1024))
    with TestClient(create_app(eng, load_tokenizer(None, eng.cfg.vocab_size), ServerConfig(model_name="tiny"))) as c:
        agg = FC.aggregate(FC.run(FC.load_dataset()[:2], FC.app_asker(c, "tiny", max_tokens=8)))
    assert agg["n"] == 2 and not any("request failed" in f["reason"] for f in agg["failures"])     # a random model answers wrongly, but it answers


def test_agent_loop_tools_sandbox_and_scoring():
    assert AG.norm_path("a/../b.txt") == "b.txt" and AG.norm_path("/x/y") == "x/y"
    for bad in ("../etc/passwd", "", "a/../../b"):
        with pytest.raises(ValueError):
            AG.norm_path(bad)
    script = {
        "sum_numbers": [_call("read_file", path="numbers.txt"), _call("write_file", path="total.txt", content="108\n"), _call("finish")],
        "rename_constant": [_call("read_file", path="config.py"), _call("read_file", path="config.py"), _call("read_file", path="nope.py"),
                            {"content": "I give up"}],
        "create_readme": [_call("write_file", path="../README.md", content="x")] * 20,
    }
    state = {}

    def ask(messages, tools):
        goal = messages[1]["content"]
        tid = next(t.id for t in AG.builtin_tasks() if t.goal == goal)
        i = state.get(tid, 0)
        state[tid] = i + 1
        assert [m["role"] for m in messages[:2]] == ["system", "user"]
        if i > 0 and messages[-1]["role"] == "tool":
            assert messages[-1]["tool_call_id"]
        return script[tid][i]
    res = AG.run_suite(ask)
    tasks = res["tasks"]
    assert tasks["sum_numbers"] == {"passed": True, "turns": 3, "reason": "finish"}
    assert not tasks["rename_constant"]["passed"] and tasks["rename_constant"]["reason"] == "the model stopped calling tools"
    assert tasks["create_readme"]["reason"] == "turn budget exhausted" and not tasks["create_readme"]["passed"]
    assert res["passed"] == 1 and res["repeated_calls"] >= 1 and res["tool_errors"] >= 2
    tr = next(t for t in res["traces"] if t.task == "rename_constant")
    assert tr.turns[2]["calls"][0]["error"] and "no such file" in tr.turns[2]["calls"][0]["result"]
    big = AG.Task("big", "read", {"big.txt": "x" * 10000}, lambda f: True, max_turns=1)
    t = AG.run_task(big, lambda m, tools: _call("read_file", path="big.txt"))
    assert t.truncated_results == 1 and t.turns[0]["calls"][0]["result"].endswith("[truncated]")


def test_requests_do_not_leak_into_each_other_and_scheduling_does_not_change_tokens():
    eng = LLMEngine(EngineArgs(model="tiny-hybrid-moe", device="cpu", max_num_seqs=4, max_model_len=256, num_kv_blocks=96))
    rep = contamination(eng, n_requests=6, rounds=2, max_tokens=10)
    assert rep["ok"] and rep["requests"] == 12
    make = lambda **kw: LLMEngine(EngineArgs(**{**dict(model="tiny-dense", device="cpu", max_num_seqs=8, max_model_len=256, num_kv_blocks=128), **kw}))
    eq = scheduler_equivalence(make, n=4, max_tokens=8)
    assert eq["ok"], eq
    assert set(eq["variants"]) == {"small_prefill_chunks", "batch_cap_2", "tbt_policy", "no_prefix_cache"}


# ----------------------------------------------------------------------------- replay gates
def test_order_comparison_names_each_way_to_fail():
    from metrale_inference_alpha_b200.bench.replay_gates import compare_orders
    a = {"s0": [1, 2, 3], "s1": [4, 5]}
    assert compare_orders([a, dict(a), dict(a)])["pass"]
    assert compare_orders([a])["why"] == "fewer than two orders"
    assert compare_orders([{}, {}])["why"] == "no samples"
    assert compare_orders([{"s0": []}, {"s0": []}])["why"] == "every reference reply is empty"
    bad = compare_orders([a, {"s0": [1, 9, 3], "s1": [4, 5]}])
    assert not bad["pass"] and bad["unequal"] == [{"sample": "s0", "order": 1, "first_difference": 1, "missing": False}]
    assert compare_orders([a, {"s0": [1, 2, 3]}])["unequal"][0]["missing"]


def test_turns_split_into_invariant_jittered_collapsed_and_unmeasured():
    from metrale_inference_alpha_b200.bench.replay_gates import ReplayScore, Turn, compare_round, compare_turn
    ref = Turn(list(range(10)), "length")
    assert compare_turn(ref, Turn(list(range(10)), "length")) == "invariant"
    assert compare_turn(ref, Turn(list(range(9)) + [99], "length")) == "jittered"           # reworded, same shape
    assert compare_turn(ref, Turn([1, 2], "length")) == "collapsed"                          # a stub: ratio 0.2
    assert compare_turn(ref, Turn(list(range(25)), "length")) == "collapsed"                 # a runaway: ratio 2.5
    assert compare_turn(ref, Turn(list(range(10)), "stop")) == "collapsed"                   # another finish reason
    assert compare_turn(ref, Turn([], None, error="boom")) == "unmeasured"
    assert compare_round([ref, ref], [ref, Turn(list(range(9)) + [7], "length")]) == "jittered"
    assert compare_round([ref, ref], [ref]) == "unmeasured"                                  # a short round
    assert compare_round([ref, ref], [Turn([1], "length"), Turn([], None, error="x")]) == "collapsed"
    ok = ReplayScore(3, ["invariant", "jittered", "invariant"]).decide()
    assert ok["pass"] and ok["jittered"] == 1
    assert "short run" in ReplayScore(3, ["invariant"]).decide()["why"]
    assert "1 collapsed" in ReplayScore(2, ["invariant", "collapsed"]).decide()["why"]
    assert "restored nothing" in ReplayScore(1, ["invariant"], zero_cache_rounds=[1]).decide()["why"]
    assert "anchors" in ReplayScore(1, ["invariant"], reference_ok=False).decide()["why"]


@pytest.mark.parametrize("model", ["tiny-dense", "tiny-hybrid-moe"])
def test_replay_gates_pass_on_the_engine(model):
    from metrale_inference_alpha_b200.bench.replay_gates import conversation_replay, decode_floor, judge_floor, order_equality
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    eng = LLMEngine(EngineArgs(model=model, device="cpu", max_num_seqs=4, max_model_len=512, num_kv_blocks=96))
    eng.scheduler.snapshot_interval = 16          # recurrent models: state snapshots (hence prefix hits) from the first block on
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(1, eng.cfg.vocab_size, (20 + 5 * i,), generator=g).tolist() for i in range(5)]
    rec = order_equality(eng, prompts, orders=3, max_tokens=8)
    assert rec.value == 1.0, rec.config
    script = [torch.randint(1, eng.cfg.vocab_size, (24,), generator=g).tolist() for _ in range(3)]
    noise_prompts = [torch.randint(1, eng.cfg.vocab_size, (30,), generator=g).tolist() for _ in range(4)]

    def noise(r):
        eng.generate([noise_prompts[r % 4]], SamplingParams(max_tokens=4, temperature=0.0))
    rec = conversation_replay(eng, script, rounds=3, max_tokens=6, noise=noise)
    assert rec.value == 1.0 and rec.config["verdicts"] == ["invariant"] * 3, rec.config
    rec = decode_floor(eng, prompts[0], floor_tok_s=0.01, runs=3, max_tokens=6)
    assert rec.config["pass"] and rec.value > 0.01
    assert not judge_floor([5.0, 6.0, 7.0], 10.0)["pass"] and not judge_floor([50.0], 10.0)["pass"]
    eng.close()


def test_gates_command_runs_the_suites_and_fails_on_an_unmet_floor(capsys):
    from metrale_inference_alpha_b200.server import cli
    cli.main(["gates", "--model", "tiny-dense", "--device", "cpu", "--rounds", "2", "--only", "order,replay,floor", "--max-num-seqs", "4"])
    out = capsys.readouterr().out
    assert out.count("PASS") == 3 and "conversation-replay" in out and "FAIL" not in out
    with pytest.raises(SystemExit):
        cli.main(["gates", "--model", "tiny-dense", "--device", "cpu", "--only", "floor", "--decode-floor", "1e9"])
    assert "under the floor" in capsys.readouterr().out


# ----------------------------------------------------------------------------- speed gates
def test_ttft_verdicts_and_baseline_rules(tmp_path):
    from metrale_inference_alpha_b200.bench.speed_gates import TtftBaselines, same_host, summarise_ttft, ttft_verdict
    assert same_host("http://localhost:8888/v1", "127.0.0.1:8888") and same_host("https://a.example", "https://A.example:443/")
    assert not same_host("http://a.example:8888", "http://a.example:9999") and not same_host("http://a", "http://b")
    s = summarise_ttft([10.0, 30.0, 20.0, None, 40.0, 50.0])
    assert s == {"n": 5, "median_ms": 30.0, "p90_ms": 50.0} and summarise_ttft([])["median_ms"] is None
    base = {"median_ms": 100.0, "p90_ms": 150.0}
    assert ttft_verdict({"median_ms": 105.0, "p90_ms": 160.0}, base) == {"verdict": "pass", "should_store": False, "why": ""}
    assert ttft_verdict({"median_ms": 90.0, "p90_ms": 140.0}, base)["should_store"]              # a better run becomes the baseline
    bad = ttft_verdict({"median_ms": 100.0, "p90_ms": 200.0}, base)
    assert bad["verdict"] == "fail" and not bad["should_store"] and "p90_ms" in bad["why"]
    assert ttft_verdict({"median_ms": 1.0, "p90_ms": 2.0}, None)["verdict"] == "no-baseline"
    assert ttft_verdict({"median_ms": 1.0, "p90_ms": 2.0}, {"median_ms": None, "p90_ms": 3.0})["verdict"] == "no-baseline"
    assert ttft_verdict({"median_ms": None, "p90_ms": None}, base)["verdict"] == "fail"
    bl = TtftBaselines(str(tmp_path / "ttft.json"))
    bl.store("http://localhost:8888", "m", "cold", base)
    again = TtftBaselines(str(tmp_path / "ttft.json"))
    assert again.find("127.0.0.1:8888", "m", "cold")["p90_ms"] == 150.0 and again.find("127.0.0.1:8888", "m", "warm") is None


def test_speed_measurements_on_the_engine(tmp_path):
    from metrale_inference_alpha_b200.bench.speed_gates import TtftBaselines, boot_memory, quick_speed, ttft_gate
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=256, num_kv_blocks=64))
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(1, eng.cfg.vocab_size, (48,), generator=g).tolist() for _ in range(4)]
    q = quick_speed(eng, prompts[0], runs=2, max_tokens=8)
    assert len(q["runs"]) == 2 and q["e2e_tok_s"] > 0 and all(r["completion_tokens"] == 8 for r in q["runs"])
    bl = TtftBaselines(str(tmp_path / "b.json"))
    first = ttft_gate(eng, prompts[1:], bl, kind="cold")
    assert first["verdict"] == "no-baseline" and first["n"] == 3 and bl.find("in-process", eng.cfg.name, "cold") is not None
    second = ttft_gate(eng, prompts[1:], bl, kind="warm", tolerance=100.0)
    assert second["verdict"] == "no-baseline" and second["kind"] == "warm"                       # warm and cold keep separate baselines
    third = ttft_gate(eng, prompts[1:], bl, kind="warm", tolerance=100.0)
    assert third["verdict"] == "pass"
    m = boot_memory(eng, warmup_prompts=prompts[:2])
    assert m["verdict"] == "info" and m["kv_blocks"] == 64 and m["weights_bytes"] > 0
    assert boot_memory(eng, budget_bytes=1)["verdict"] == "fail"
    eng.close()
