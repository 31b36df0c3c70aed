"""Request shaping and the HTTP surface on CPU: tokenizer + streaming detokeniser, chat
template, reasoning split, tool-call parsers (with salvage and schema coercion), JSON
grammar, rate limiter, levers, telemetry, CLI, and every route of the app driven through
FastAPI's test client over the tiny dense model. Mirrors the reference's server test
strategy (``crates/server/tests``: golden request / response shapes, SSE framing, auth)."""
import json
import re
import time

import pytest
import torch

from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.server.chat_template import ChatRenderer
from metrale_inference_alpha_b200.server.grammar import (JsonMatcher, TokenGrammar, grammar_for_response_format,
                                                           validate_schema)
from metrale_inference_alpha_b200.server.ratelimit import RateLimiter
from metrale_inference_alpha_b200.server.reasoning_parser import ReasoningParser, split_reasoning
from metrale_inference_alpha_b200.server.tokenizer import ByteTokenizer, IncrementalDetokenizer, load_tokenizer
from metrale_inference_alpha_b200.server.tool_parser import StreamingToolDetector, parse_tool_calls
from metrale_inference_alpha_b200.utils import levers
from metrale_inference_alpha_b200.utils.telemetry import Telemetry

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}}}]


# ---------------------------------------------------------------------------- tokenizer
def test_byte_tokenizer_roundtrip_and_incremental_utf8():
    tk = ByteTokenizer(4096)
    s = "héllo wörld ✓ 你好"
    ids = tk.encode(s)
    assert tk.decode(ids) == s
    d = IncrementalDetokenizer(tk)
    out = "".join(d.push([i]) for i in ids) + d.flush()
    assert out == s                                   # multi-byte characters never split
    assert load_tokenizer(None, 512).vocab_size == 512


# ---------------------------------------------------------------------------- templates
def test_chat_template_default_and_custom():
    r = ChatRenderer()
    txt = r.render([{"role": "system", "content": "be brief"},
                    {"role": "user", "content": [{"type": "text", "text": "hi"}, {"type": "text", "text": " there"}]}])
    assert "be brief" in txt and "hi there" in txt and txt.rstrip().endswith("assistant")
    with_tools = r.render([{"role": "user", "content": "x"}], tools=TOOLS)
    assert "get_weather" in with_tools
    custom = ChatRenderer("{% for m in messages %}[{{ m.role }}]{{ m.content }}{% endfor %}{% if add_generation_prompt %}[a]{% endif %}")
    assert custom.render([{"role": "user", "content": "q"}]) == "[user]q[a]"


# ---------------------------------------------------------------------------- reasoning
def test_reasoning_split_whole_and_streamed_by_character():
    text = "<think>step one\nstep two</think>The answer is 4."
    assert split_reasoning(text) == ("step one\nstep two", "The answer is 4.")
    p = ReasoningParser()
    r = c = ""
    for ch in text:
        a, b = p.push(ch)
        r, c = r + a, c + b
    a, b = p.flush()
    assert (r + a, c + b) == ("step one\nstep two", "The answer is 4.")
    # template already opened the block
    assert split_reasoning("inner</think>outer", starts_open=True) == ("inner", "outer")
    assert split_reasoning("no tags at all") == ("", "no tags at all")
    assert split_reasoning("never closes", starts_open=True) == ("never closes", "")


# ---------------------------------------------------------------------------- tool calls
def test_tool_parsers_primary_and_salvage():
    hermes = 'Sure.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo", "days": "3"}}\n</tool_call>'
    rest, calls = parse_tool_calls(hermes, "hermes", TOOLS)
    assert rest == "Sure." and len(calls) == 1
    args = json.loads(calls[0]["function"]["arguments"])
    assert args == {"city": "Oslo", "days": 3}        # "3" coerced to the declared integer
    assert calls[0]["id"].startswith("call_") and calls[0]["type"] == "function"

    xml = "<tool_call>\n<function=get_weather>\n<parameter=city>\nRome\n</parameter>\n</function>\n</tool_call>"
    _, calls = parse_tool_calls(xml, "qwen3_xml", TOOLS)
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Rome"}
    _, calls = parse_tool_calls(xml, "hermes", TOOLS)               # wrong primary parser: salvaged
    assert calls and calls[0]["function"]["name"] == "get_weather"

    mistral = '[TOOL_CALLS] [{"name": "get_weather", "arguments": {"city": "Lima"}}]'
    _, calls = parse_tool_calls(mistral, "mistral", TOOLS)
    assert json.loads(calls[0]["function"]["arguments"])["city"] == "Lima"

    bare = 'I will call {"name": "get_wether", "arguments": {"city": "Kyiv"}} now'
    rest, calls = parse_tool_calls(bare, "hermes", TOOLS)
    assert calls[0]["function"]["name"] == "get_weather"             # fuzzy name repair
    assert "{" not in rest

    assert parse_tool_calls("plain text", "hermes", TOOLS) == ("plain text", [])
    thought = '<think>{"name": "get_weather", "arguments": {}}</think>done'
    assert parse_tool_calls(thought, "hermes", TOOLS)[1] == []       # reasoning is not scanned


def test_streaming_tool_detector_holds_back_markup():
    d = StreamingToolDetector()
    seen = ""
    for ch in 'ok <tool_call>{"name": "f", "arguments": {}}</tool_call>':
        seen += d.push(ch)
    assert seen == "ok " and d.finish().startswith("<tool_call>")
    d = StreamingToolDetector()
    assert "".join(d.push(ch) for ch in "a < b and <tool") + d.finish() == "a < b and <tool"


# ---------------------------------------------------------------------------- grammar
@pytest.mark.parametrize("doc,ok", [
    ('{"a": 1, "b": [true, null, -2.5e3], "c": {"d": "x\\n\\u00e9"}}', True),
    ('  {"k": ""}  ', True), ('{}', True), ('{"a": 01}', False), ('{"a": 1,}', False),
    ('{a: 1}', False), ('{"a": tru}', False), ('{"a": "x}', False), ('[1, 2]', False)])
def test_json_matcher_accepts_exactly_valid_objects(doc, ok):
    m = JsonMatcher(require_object=True)
    fed = m.feed_bytes(doc.encode())
    assert (fed and m.is_complete()) == ok


def test_token_grammar_drives_a_random_model_to_valid_json():
    tk = ByteTokenizer(512)
    g = TokenGrammar(tk, JsonMatcher(require_object=True), eos_token_id=0)
    gen = torch.Generator().manual_seed(3)
    out = []
    for _ in range(400):
        logits = torch.randn(512, generator=gen)
        if len(out) > 40:
            logits[0] += 50.0                        # the model "wants" to stop
            logits[ord("}")] += 20.0
            logits[ord('"')] += 10.0
        g.observe_logits(logits)
        mask = g.allowed_mask(512)
        assert mask.any()
        t = int(torch.where(mask, logits, torch.full_like(logits, -1e30)).argmax())
        if t == 0:
            break
        g.advance(t)
        out.append(t)
    doc = tk.decode(out)
    assert isinstance(json.loads(doc), dict)
    assert grammar_for_response_format({"type": "text"}, tk) is None
    assert grammar_for_response_format({"type": "json_object"}, tk, 0) is not None


def test_validate_schema_subset():
    sch = {"type": "object", "required": ["n"], "properties": {"n": {"type": "integer"}, "t": {"enum": ["a", "b"]},
                                                               "l": {"type": "array", "items": {"type": "number"}}}}
    assert validate_schema({"n": 1, "t": "a", "l": [1, 2.5]}, sch)
    assert not validate_schema({"t": "a"}, sch)
    assert not validate_schema({"n": True}, sch)
    assert not validate_schema({"n": 1, "t": "z"}, sch)
    assert not validate_schema({"n": 1, "l": ["x"]}, sch)
    assert validate_schema(3, {"anyOf": [{"type": "string"}, {"type": "integer"}]})


# ---------------------------------------------------------------------------- small utilities
def test_rate_limiter_token_bucket():
    t = [0.0]
    rl = RateLimiter(2.0, burst=2, clock=lambda: t[0])
    assert rl.allow("k") and rl.allow("k") and not rl.allow("k")
    assert rl.allow("other")
    t[0] = 0.6
    assert rl.allow("k") and not rl.allow("k")
    assert RateLimiter(0.0).allow("x")


def test_undeclared_levers_are_refused():
    assert levers.undeclared({"METRALE_PDL": "1", "PATH": "/bin"}) == []
    assert levers.undeclared({"METRALE_PDLL": "1"}) == ["METRALE_PDLL"]
    with pytest.raises(SystemExit):
        levers.check_environment({"METRALE_TYPO": "1"})


def test_telemetry_kernel_level_without_a_gpu_falls_back_to_host_timers():
    """Level "kernel" (alias "full") installs CUDA-event spans and the per-launch hook only on a
    CUDA device; without one it behaves like "basic" and leaves the launch hook alone."""
    from metrale_inference_alpha_b200.ops import _native
    t = Telemetry("full")
    assert t.level == "kernel" and t.enabled
    assert _native._launch_hook is None or torch.cuda.is_available()
    with t.span("lane"):
        pass
    assert "metrale_lane_ms_count 1" in t.prometheus()
    t.close()


def test_telemetry_prometheus_text():
    t = Telemetry("basic")
    t.inc("requests")
    t.inc("requests", 2)
    t.set("queue_depth", 5)
    t.observe_ms("step", 2.0)
    t.observe_ms("step", 4.0)
    with t.span("load"):
        pass
    text = t.prometheus({"engine_steps": 7})
    assert "metrale_requests_total 3" in text and "metrale_queue_depth 5" in text and "metrale_engine_steps 7" in text
    assert "step" in text
    off = Telemetry("off")
    off.inc("x")
    assert "metrale_x_total" not in off.prometheus()


def test_cli_dump_options_and_doctor():
    from metrale_inference_alpha_b200.server import cli
    opts = cli.dump_serve_options()
    assert "--port" in opts and "--max-num-seqs" in opts and "METRALE_PDL" in opts["__env_levers__"]
    rep = cli.doctor()
    assert "torch" in rep and "native_library" in rep
    ns = cli.build_parser().parse_args(["serve", "--model", "tiny-dense", "--max-num-seqs", "4", "--no-use-cuda-graphs"])
    ea = cli._engine_args(ns)
    assert ea.max_num_seqs == 4 and ea.use_cuda_graphs is False


def test_bench_ladder_on_cpu():
    from metrale_inference_alpha_b200.bench.ladder import run_ladder
    rows = run_ladder(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=128), [1, 3], isl=12, osl=6)
    assert [r["concurrency"] for r in rows] == [1, 3]
    assert rows[1]["tokens"] == 18 and rows[1]["tok_s"] > 0 and rows[1]["ttft_p50_ms"] > 0


# ---------------------------------------------------------------------------- HTTP surface
@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=8, max_model_len=512))
    tok = load_tokenizer(None, eng.cfg.vocab_size)
    app = create_app(eng, tok, ServerConfig(model_name="tiny", auth_tokens=["sekret"]))
    with TestClient(app) as c:
        c.headers.update({"Authorization": "Bearer sekret"})
        yield c


def test_health_models_auth(client):
    assert client.get("/health").json()["status"] == "ok"
    assert client.get("/health/live").status_code == 200
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    r = client.get("/v1/models", headers={"Authorization": "Bearer wrong"})
    assert r.status_code == 401 and r.json()["error"]["type"] == "authentication_error"
    assert client.get("/v1/models", headers={"Authorization": "", "x-api-key": "sekret"}).status_code == 200


def test_chat_completion_shape_usage_and_determinism(client):
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 8, "temperature": 0, "return_token_ids": True}
    a = client.post("/v1/chat/completions", json=body).json()
    b = client.post("/v1/chat/completions", json=body).json()
    assert a["object"] == "chat.completion" and a["choices"][0]["finish_reason"] == "length"
    assert a["choices"][0]["token_ids"] == b["choices"][0]["token_ids"] and len(a["choices"][0]["token_ids"]) == 8
    u = a["usage"]
    assert u["completion_tokens"] == 8 and u["total_tokens"] == u["prompt_tokens"] + 8
    for k in ("time_to_first_token_ms", "decode_time_ms", "total_time_ms", "response_tokens_per_second"):
        assert k in u
    assert b["usage"]["prompt_tokens_details"]["cached_tokens"] > 0      # second call hits the prefix cache
    assert client.post("/v1/chat/completions", json={"max_tokens": 1}).status_code == 400


def test_chat_streaming_sse_framing(client):
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "stream": True,
            "stream_options": {"include_usage": True}}
    with client.stream("POST", "/v1/chat/completions", json=body) as s:
        lines = [l for l in s.iter_lines() if l]
    assert all(l.startswith("data: ") for l in lines) and lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == 5
    assert chunks[-2]["choices"][0]["finish_reason"] == "length"


def test_completions_logprobs_stop_and_stream(client):
    r = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 6, "logprobs": True, "return_token_ids": True}).json()
    ch = r["choices"][0]
    assert len(ch["token_ids"]) == 6 and len(ch["logprobs"]["token_logprobs"]) == 6
    assert all(lp <= 0 for lp in ch["logprobs"]["token_logprobs"])
    r = client.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 3}).json()
    assert r["usage"]["prompt_tokens"] == 3
    with client.stream("POST", "/v1/completions", json={"prompt": "abc", "max_tokens": 3, "stream": True}) as s:
        lines = [l for l in s.iter_lines() if l]
    assert lines[-1] == "data: [DONE]" and "usage" in json.loads(lines[-2][6:])


def test_sampling_fields_reach_the_sampler(client):
    body = {"prompt": "xyz", "max_tokens": 6, "temperature": 0.9, "top_p": 0.9, "top_k": 20, "seed": 11,
            "repetition_penalty": 1.1, "presence_penalty": 0.2, "return_token_ids": True}
    a = client.post("/v1/completions", json=body).json()["choices"][0]["token_ids"]
    b = client.post("/v1/completions", json=body).json()["choices"][0]["token_ids"]
    assert a == b                                    # seeded sampling is reproducible
    body["seed"] = 12
    c = client.post("/v1/completions", json=body).json()["choices"][0]["token_ids"]
    assert len(c) == 6


def test_json_mode_returns_a_json_object(client):
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "json please"}],
                                                  "max_tokens": 48, "response_format": {"type": "json_object"},
                                                  "temperature": 0}).json()
    text = r["choices"][0]["message"]["content"]
    m = JsonMatcher(require_object=True)
    assert m.feed_bytes(text.encode())               # always a legal prefix of a JSON object
    if r["choices"][0]["finish_reason"] == "stop":
        assert isinstance(json.loads(text), dict)


def test_json_schema_regex_and_tool_grammar_constrain_the_output(client):
    from metrale_inference_alpha_b200 import grammar as G
    schema = {"type": "object", "properties": {"n": {"type": "integer", "minimum": 0}, "k": {"enum": ["a", "b"]}},
              "required": ["n", "k"]}
    msgs = [{"role": "user", "content": "go"}]
    r = client.post("/v1/chat/completions", json={
        "messages": msgs, "max_tokens": 40, "temperature": 0,
        "response_format": {"type": "json_schema", "json_schema": {"name": "x", "schema": schema}}}).json()
    text = r["choices"][0]["message"]["content"]
    m = G.GrammarMatcher(G.compile_json_schema(schema))
    assert m.feed_bytes(text.encode())                       # a legal prefix of a document of this schema
    if r["choices"][0]["finish_reason"] == "stop":
        v = json.loads(text)
        assert v["n"] >= 0 and v["k"] in ("a", "b")
    r = client.post("/v1/chat/completions", json={
        "messages": msgs, "max_tokens": 24, "temperature": 0.8, "seed": 5,
        "response_format": {"type": "regex", "pattern": r"(yes|no)( [a-z]{1,3}){0,2}\."}}).json()
    text = r["choices"][0]["message"]["content"]
    assert G.GrammarMatcher(G.compile_regex(r"(yes|no)( [a-z]{1,3}){0,2}\.")).feed_bytes(text.encode())
    assert r["choices"][0]["finish_reason"] == "stop"         # the pattern is finite: the mask ends it
    import re as _re
    assert _re.fullmatch(r"(yes|no)( [a-z]{1,3}){0,2}\.", text)
    tools = [{"type": "function", "function": {"name": "f", "parameters": {
        "type": "object", "properties": {"x": {"type": "boolean"}}, "required": ["x"]}}}]
    r = client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 64, "temperature": 0,
                                                  "tools": tools, "tool_choice": "required"}).json()
    ch = r["choices"][0]
    if ch["finish_reason"] == "tool_calls":
        call = ch["message"]["tool_calls"][0]["function"]
        assert call["name"] == "f" and isinstance(json.loads(call["arguments"])["x"], bool)
    r = client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 4,
                                                  "response_format": {"type": "regex", "pattern": "(a"}})
    assert r.status_code == 400 and "invalid grammar" in r.text


def test_anthropic_messages_and_count_tokens(client):
    body = {"model": "tiny", "max_tokens": 5, "system": "be brief", "messages": [{"role": "user", "content": "hi"}]}
    r = client.post("/v1/messages", json=body).json()
    assert r["type"] == "message" and r["role"] == "assistant" and r["stop_reason"] == "max_tokens"
    assert r["usage"]["output_tokens"] == 5 and r["usage"]["input_tokens"] > 0
    n = client.post("/v1/messages/count_tokens", json=body).json()["input_tokens"]
    assert n == r["usage"]["input_tokens"]
    assert client.post("/v1/messages", json={"messages": []}).status_code == 400
    with client.stream("POST", "/v1/messages", json=dict(body, stream=True)) as s:
        events = [l[7:] for l in s.iter_lines() if l.startswith("event: ")]
    assert events[0] == "message_start" and events[-1] == "message_stop" and "message_delta" in events


def test_responses_api(client):
    r = client.post("/v1/responses", json={"input": "hi", "instructions": "short", "max_output_tokens": 4}).json()
    assert r["object"] == "response" and r["status"] == "completed"
    assert r["output"][-1]["type"] == "message" and r["usage"]["output_tokens"] == 4


def test_tokenize_metrics_config_memory(client):
    t = client.post("/tokenize", json={"prompt": "abc"}).json()
    assert t["count"] == 3 and client.post("/detokenize", json={"tokens": t["tokens"]}).json()["prompt"] == "abc"
    m = client.get("/metrics").text
    assert "metrale_http_requests_total" in m and "metrale_engine_decode_tokens" in m
    cfg = client.get("/serve-config").json()
    assert cfg["engine"]["max_num_seqs"] == 8 and cfg["model_config"]["num_layers"] >= 1
    mem = client.get("/memory").json()
    assert mem["kv_bytes"] > 0 and mem["weights_bytes"] > 0


def test_gpu_fault_latch_turns_routes_into_503(client):
    eng = client.app.state.engine
    eng.fault.set("injected on the host")
    try:
        assert client.get("/health").status_code == 503
        r = client.post("/v1/completions", json={"prompt": "a", "max_tokens": 1})
        assert r.status_code == 503 and r.json()["error"]["type"] == "gpu_fault"
        assert client.get("/health/live").status_code == 200
    finally:
        eng.fault._reason = None if hasattr(eng.fault, "_reason") else None
        eng.fault.__init__()
    assert client.get("/health").status_code == 200


def test_more_tool_call_formats():
    d = "｜DSML｜"
    cases = {
        "minimax_xml": 'ok <minimax:tool_call>\n<invoke name="get_weather">\n<parameter name="city">Oslo</parameter>\n'
                       '<parameter name="days">3</parameter>\n</invoke>\n</minimax:tool_call>',
        "gemma4": '<|tool_call>call:get_weather{city:"Oslo",days:3}<tool_call|>',
        "deepseek_v4_dsml": f'<{d}tool_calls>\n<{d}invoke name="get_weather">\n<{d}parameter name="city" string="true">Oslo'
                            f'</{d}parameter>\n<{d}parameter name="days" string="false">3</{d}parameter>\n</{d}invoke>\n</{d}tool_calls>',
        "poolside_v1": '<tool_call>get_weather<arg_key>city</arg_key><arg_value>Oslo</arg_value>'
                       '<arg_key>days</arg_key><arg_value>3</arg_value></tool_call>',
    }
    for fmt, text in cases.items():
        rest, calls = parse_tool_calls(text, fmt, TOOLS)
        assert len(calls) == 1 and calls[0]["function"]["name"] == "get_weather", fmt
        assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo", "days": 3}, fmt
        assert "tool_call" not in rest and "DSML" not in rest
    # poolside: bare name = zero-argument call; a repeated key drops the call
    assert parse_tool_calls("<tool_call>get_weather</tool_call>", "poolside_v1", TOOLS)[1][0]["function"]["arguments"] == "{}"
    dup = '<tool_call>get_weather<arg_key>a</arg_key><arg_value>1</arg_value><arg_key>a</arg_key><arg_value>2</arg_value></tool_call>'
    assert parse_tool_calls(dup, "poolside_v1", TOOLS)[1] == []
    # DSML: a repeated key drops the invoke whole
    bad = (f'<{d}tool_calls><{d}invoke name="get_weather"><{d}parameter name="city" string="true">a</{d}parameter>'
           f'<{d}parameter name="city" string="true">b</{d}parameter></{d}invoke></{d}tool_calls>')
    assert parse_tool_calls(bad, "deepseek_v4_dsml", TOOLS)[1] == []


def test_reasoning_formats_mistral_and_gemma():
    assert split_reasoning("[THINK]plan[/THINK]answer", "mistral") == ("plan", "answer")
    assert split_reasoning("<|channel>plan<channel|>answer", "gemma4") == ("plan", "answer")


def test_responses_store_and_previous_response_id(client):
    a = client.post("/v1/responses", json={"input": "first question", "max_output_tokens": 3}).json()
    b = client.post("/v1/responses", json={"input": "follow up", "previous_response_id": a["id"], "max_output_tokens": 3}).json()
    assert b["previous_response_id"] == a["id"]
    assert b["usage"]["input_tokens"] > a["usage"]["input_tokens"]        # the thread was prepended
    assert client.get(f"/v1/responses/{a['id']}").json()["id"] == a["id"]
    assert client.post("/v1/responses", json={"input": "x", "previous_response_id": "resp_nope"}).status_code == 404
    assert client.delete(f"/v1/responses/{b['id']}").json()["deleted"] is True
    assert client.get(f"/v1/responses/{b['id']}").status_code == 404
    c = client.post("/v1/responses", json={"input": "not stored", "store": False, "max_output_tokens": 2}).json()
    assert client.get(f"/v1/responses/{c['id']}").status_code == 404


def test_nvml_sampler_against_a_fake_binding():
    from types import SimpleNamespace
    from metrale_inference_alpha_b200.utils.nvml import DeviceSampler, decode_reasons
    power = iter([400_000, 600_000, 800_000])

    class Fake:
        NVML_CLOCK_SM, NVML_CLOCK_MEM, NVML_TEMPERATURE_GPU = 1, 2, 0
        nvmlInit = staticmethod(lambda: None)
        nvmlDeviceGetHandleByIndex = staticmethod(lambda i: "h")
        nvmlDeviceGetClockInfo = staticmethod(lambda h, k: 1965 if k == 1 else 3996)
        nvmlDeviceGetPowerUsage = staticmethod(lambda h: next(power))
        nvmlDeviceGetTemperature = staticmethod(lambda h, k: 55)
        nvmlDeviceGetUtilizationRates = staticmethod(lambda h: SimpleNamespace(gpu=97))
        nvmlDeviceGetMemoryInfo = staticmethod(lambda h: SimpleNamespace(used=10 << 30))
        nvmlDeviceGetCurrentClocksThrottleReasons = staticmethod(lambda h: 0x4)
    t = iter([0.0, 1.0, 2.0])
    s = DeviceSampler(nvml=Fake, clock=lambda: next(t))
    for _ in range(3):
        s.sample_once()
    out = s.summary(tokens=100)
    assert out["energy_j"] == pytest.approx(500.0 + 700.0) and out["joules_per_token"] == pytest.approx(12.0)
    assert out["reasons"] == ["sw_power_cap"] and out["rejected"] is False and out["sm_mhz_median"] == 1965
    assert decode_reasons(0x8 | 0x40) == ["hw_slowdown", "hw_thermal_slowdown"]


def test_forced_think_close_and_budget_over_http(tmp_path):
    from metrale_inference_alpha_b200.sampling.host import forced_think_close
    end = [7, 8, 9]
    assert forced_think_close([1, 2], 4, end) is None                     # under budget
    assert forced_think_close([1, 2, 3, 4], 4, end) == 7
    assert forced_think_close([1, 2, 3, 4, 7], 4, end) == 8               # resumes a partly written marker
    assert forced_think_close([1, 2, 3, 4, 7, 8], 4, end) == 9
    assert forced_think_close([1, 2, 3, 4, 7, 8, 9, 5, 5], 4, end) is None  # closed: free again
    assert forced_think_close([7, 8, 9, 1, 2, 3], 4, end) is None
    assert forced_think_close([1, 2, 3, 7], 4, end) == 7                  # a 7 before the budget is not progress
    from fastapi.testclient import TestClient
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=512))
    tok = load_tokenizer(None, eng.cfg.vocab_size)
    cfg = ServerConfig(model_name="tiny", max_thinking_budget=6, dump_dir=str(tmp_path / "dump"),
                       default_min_p=0.05, content_loop_watchdog=0.5)
    with TestClient(create_app(eng, tok, cfg)) as c:
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "think"}], "max_tokens": 40,
                                                 "temperature": 0, "enable_thinking": True,
                                                 "thinking_token_budget": 1000, "return_token_ids": True}).json()
        ids = r["choices"][0]["token_ids"]
        close = tok.encode("</think>")
        assert ids[6:6 + len(close)] == close                             # the server cap (6) beat the request's 1000
        assert "</think>" not in r["choices"][0]["message"].get("content", "")
        assert r["choices"][0]["message"].get("reasoning_content")
    dumps = sorted((tmp_path / "dump").glob("*.json"))
    assert len(dumps) == 1
    d = json.loads(dumps[0].read_text())
    assert d["path"] == "/v1/chat/completions" and d["status"] == 200 and d["request"]["thinking_token_budget"] == 1000


def test_serve_alias_flags(tmp_path):
    from metrale_inference_alpha_b200.server.cli import apply_aliases, build_parser
    tf = tmp_path / "tokens.txt"
    tf.write_text("# comment\nalpha\n\nbeta\n")
    ns = build_parser().parse_args(["serve", "--bind", "0.0.0.0:9001", "--model-name", "m", "--max-seq-len", "777",
                                    "--max-batch-size", "9", "--request-timeout", "12", "--auth-token", "gamma",
                                    "--auth-tokens-file", str(tf), "--require-auth", "--ngram-speculative",
                                    "--kv-cache-dtype", "fp8", "--oom-guard-mb", "1024"])
    apply_aliases(ns)
    assert (ns.host, ns.port, ns.served_model_name) == ("0.0.0.0", 9001, "m")
    assert (ns.max_model_len, ns.max_num_seqs, ns.request_timeout_s, ns.speculative) == (777, 9, 12.0, "ngram")
    assert ns.api_key == ["gamma", "alpha", "beta"] and ns.kv_cache_dtype == "fp8" and ns.oom_guard_mb == 1024
    ns = build_parser().parse_args(["serve", "--require-auth"])
    with pytest.raises(SystemExit):
        apply_aliases(ns)
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=2, max_model_len=128, kv_cache_dtype="fp8"))
    assert eng.cfg.kv_dtype == "fp8"
    assert len(eng.generate([[1, 2, 3]], __import__("metrale_inference_alpha_b200").sampling.params.SamplingParams(max_tokens=3))[0].output_ids) == 3


def test_conversations_stored_completions_stubs_and_introspection(client):
    # 501 stubs carry an OpenAI-shaped error, not a 404
    for method, path in [("post", "/v1/embeddings"), ("post", "/v1/audio/speech"), ("get", "/v1/files"),
                         ("post", "/v1/images/generations"), ("post", "/v1/moderations"), ("get", "/v1/batches/b1")]:
        r = getattr(client, method)(path)
        assert r.status_code == 501 and r.json()["error"]["code"] == "not_implemented", path
    # conversations: create, add, list (desc by default), get / delete items, metadata rules
    c = client.post("/v1/conversations", json={"metadata": {"topic": "x"},
                                               "items": [{"type": "message", "role": "user", "content": "hello"}]}).json()
    cid = c["id"]
    assert cid.startswith("conv_") and c["metadata"] == {"topic": "x"} and "items" not in c
    new = client.post(f"/v1/conversations/{cid}/items", json={"items": [
        {"role": "assistant", "content": "hi there"}, {"type": "function_call", "name": "f", "arguments": "{}", "call_id": "c1"},
        {"type": "function_call_output", "call_id": "c1", "output": "42"}]}).json()
    assert len(new["data"]) == 3 and new["data"][0]["content"][0]["type"] == "output_text"
    lst = client.get(f"/v1/conversations/{cid}/items?limit=2").json()
    assert len(lst["data"]) == 2 and lst["has_more"] and lst["data"][0]["type"] == "function_call_output"
    asc = client.get(f"/v1/conversations/{cid}/items?order=asc&limit=100").json()["data"]
    assert [i["type"] for i in asc] == ["message", "message", "function_call", "function_call_output"]
    iid = asc[1]["id"]
    assert client.get(f"/v1/conversations/{cid}/items/{iid}").json()["role"] == "assistant"
    assert client.delete(f"/v1/conversations/{cid}/items/{iid}").status_code == 200
    assert client.get(f"/v1/conversations/{cid}/items/{iid}").status_code == 404
    r = client.post("/v1/conversations", json={"items": [{"role": "user", "content": "x"}] * 21})
    assert r.status_code == 400 and r.json()["error"]["code"] == "items_too_many"
    assert client.post(f"/v1/conversations/{cid}", json={"metadata": {"k": 1}}).status_code == 400
    assert client.post(f"/v1/conversations/{cid}", json={"metadata": {"k": "v"}}).json()["metadata"] == {"k": "v"}
    # /v1/responses continues a conversation and appends to it
    before = len(client.get(f"/v1/conversations/{cid}/items?order=asc&limit=100").json()["data"])
    r = client.post("/v1/responses", json={"input": "and now?", "conversation": cid, "max_output_tokens": 4}).json()
    assert r["status"] == "completed"
    after = client.get(f"/v1/conversations/{cid}/items?order=asc&limit=100").json()["data"]
    assert len(after) == before + 2 and after[-2]["role"] == "user" and after[-1]["role"] == "assistant"
    items = client.get(f"/v1/responses/{r['id']}/input_items").json()
    assert items["data"][0]["content"][0]["text"] == "and now?"
    assert client.post(f"/v1/responses/{r['id']}/cancel").status_code == 400        # already completed
    assert client.post("/v1/responses/resp_nope/cancel").status_code == 404
    assert client.post("/v1/responses", json={"input": "x", "conversation": cid, "previous_response_id": r["id"]}).status_code == 400
    assert client.delete(f"/v1/conversations/{cid}").json()["deleted"] and client.get(f"/v1/conversations/{cid}").status_code == 404
    # stored chat completions
    a = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                                  "store": True, "metadata": {"run": "7"}}).json()
    got = client.get(f"/v1/chat/completions/{a['id']}").json()
    assert got["choices"] == a["choices"] and got["metadata"] == {"run": "7"}
    assert client.get("/v1/chat/completions/chatcmpl-unknown").status_code == 404
    # model lookup, LoRA control, introspection
    assert client.get("/v1/models/tiny").json()["id"] == "tiny"
    assert client.get("/v1/models/org/other-model").json()["error"]["code"] == "model_not_found"
    assert client.post("/v1/lora/active", json={"name": "nope"}).status_code == 404
    assert client.post("/v1/lora/active", json={"name": None}).json() == {"active": None}
    assert client.post("/v1/lora/load", json={"name": "x"}).status_code == 400
    assert client.post("/v1/lora/load", json={"name": "x", "path": "/nonexistent/adapter"}).status_code == 400
    fw = client.get("/forward").json()
    assert fw["arch"] == "dense_gqa" and fw["kv_dtype"] in ("bf16", "fp8") and fw["max_num_seqs"] == 8
    hw = client.get("/hardware").json()
    assert "devices" in hw and "torch" in hw
    with client.stream("GET", "/v1/events?limit=2") as s:
        frames = [json.loads(l[6:]) for l in s.iter_lines() if l.startswith("data: ")]
    assert [f["seq"] for f in frames] == [0, 1] and "counters" in frames[0] and "engine" in frames[0]
    big = client.post("/v1/chat/completions", content=b"x", headers={"content-length": str(64 << 20)})
    assert big.status_code in (400, 413)


def test_model_library_resolve_plan_and_download_with_resume(tmp_path):
    import http.server
    import threading

    from metrale_inference_alpha_b200.server import model_library as ML
    # ---- plan: only contained metadata / safetensors names, small first, weights last
    files = [ML.RemoteFile(n, s) for n, s in [
        ("model-00002.safetensors", 300), ("model-00001.safetensors", 500), ("config.json", 40), ("pytorch_model.bin", 999),
        ("../evil.safetensors", 1), ("onnx/model.safetensors", 5), ("README.md", 10), ("tokenizer.json", 80),
        ("sub/config.json", 1), ("model.safetensors.index.json", 20), ("C:evil.safetensors", 1), ("a//b.safetensors", 1)]]
    assert [f.name for f in ML.select(files)] == ["config.json", "tokenizer.json", "model.safetensors.index.json",
                                                   "model-00002.safetensors", "model-00001.safetensors"]
    # ---- a Hub-shaped server over a directory
    repo, sha = "org/tiny-model", "abc123"
    content = {"config.json": b'{"model_type":"llama"}', "tokenizer.json": b"{}", "model.safetensors": bytes(range(256)) * 4096,
               "pytorch_model.bin": b"zzz"}
    ranges = []

    class H(http.server.BaseHTTPRequestHandler):
        def do_GET(self):
            if self.path.startswith(f"/api/models/{repo}/revision/main"):
                body = json.dumps({"sha": sha, "siblings": [{"rfilename": n, "size": len(b)} for n, b in content.items()]}).encode()
                self.send_response(200)
            elif self.path.startswith(f"/{repo}/resolve/{sha}/"):
                data = content.get(self.path.split(f"/resolve/{sha}/", 1)[1])
                if data is None:
                    self.send_response(404)
                    self.end_headers()
                    return
                rng = self.headers.get("Range")
                if rng:
                    start = int(rng.split("=")[1].split("-")[0])
                    ranges.append(start)
                    body = data[start:]
                    self.send_response(206)
                else:
                    body = data
                    self.send_response(200)
            else:
                self.send_response(404)
                self.end_headers()
                return
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def log_message(self, *a):
            pass
    srv = http.server.HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    ep = f"http://127.0.0.1:{srv.server_port}"
    cache = tmp_path / "hub"
    try:
        with pytest.raises(ML.ModelNotFound, match="download it first"):
            ML.resolve_model_dir(repo, str(cache))
        # a previous attempt left half of the weights behind: the download resumes it
        snap = ML.repo_dir(cache, repo) / "snapshots" / sha
        snap.mkdir(parents=True)
        (snap / "model.safetensors.part").write_bytes(content["model.safetensors"][:300000])
        with pytest.raises(ML.ModelNotFound, match="no default revision"):
            ML.resolve_model_dir(repo, str(cache))                 # refs/main is not published yet
        seen = []
        path = ML.download(repo, str(cache), ep, progress=lambda n, d, t: seen.append((n, d, t)))
        assert path == str(snap) and ranges == [300000]
        assert (snap / "model.safetensors").read_bytes() == content["model.safetensors"]
        assert not (snap / "pytorch_model.bin").exists() and not (snap / "model.safetensors.part").exists()
        assert seen[-1][1] == seen[-1][2] - 300000 or seen[-1][1] <= seen[-1][2]
        assert ML.resolve_model_dir(repo, str(cache)) == str(snap)
        assert ML.resolve_model_dir("tiny-dense", str(cache), presets=("tiny-dense",)) == "tiny-dense"
        assert ML.resolve_model_dir(str(snap)) == str(snap)
        rows = ML.list_models(str(cache))
        assert rows == [{"repo": repo, "revision": sha, "bytes": rows[0]["bytes"], "complete": True}] and rows[0]["bytes"] > 1 << 20
        ML.download(repo, str(cache), ep)                          # second run: nothing to fetch
        assert ranges == [300000]
        with pytest.raises(ML.DownloadError, match="HTTP 404"):
            ML.download("org/missing", str(cache), ep)
    finally:
        srv.shutdown()
    with pytest.raises(ML.DownloadError, match="cannot reach"):
        ML.download(repo, str(tmp_path / "c2"), "http://127.0.0.1:9")


class _ClientTransport:
    """The TUI's transport over an in-process TestClient."""

    def __init__(self, client):
        self.c = client

    def get_text(self, path):
        r = self.c.get(path)
        if r.status_code != 200:
            raise RuntimeError(f"HTTP {r.status_code}")
        return r.text

    def post_stream(self, path, body):
        with self.c.stream("POST", path, json=body) as s:
            yield from s.iter_lines()


def test_tui_dashboard_and_chat_against_the_app(client, tmp_path):
    from rich.console import Console

    from metrale_inference_alpha_b200.server import tui
    m = tui.parse_prometheus('# c\nmetrale_x_total 5\nmetrale_h_ms_bucket{le="10"} 2\nmetrale_h_ms_bucket{le="20"} 6\n'
                             'metrale_h_ms_bucket{le="+Inf"} 8\nbroken line here\nmetrale_y 1e3\n')
    assert m["metrale_x_total"] == 5 and m["metrale_y"] == 1000 and len(m) == 5
    assert abs(tui.histogram_quantile(m, "metrale_h_ms", 0.5) - 15.0) < 1e-6         # 4th of 8: halfway through (10, 20]
    assert tui.histogram_quantile(m, "metrale_h_ms", 0.99) == 20.0                    # lands in +Inf: last finite bound
    assert tui.histogram_quantile(m, "metrale_nope", 0.5) is None
    assert tui.sparkline([]) == "(no samples yet)" and tui.sparkline([0, 5, 10]).startswith("▁▄█")
    tr = _ClientTransport(client)
    now = [100.0]
    dash = tui.Dashboard(tr, clock=lambda: now[0])
    dash.poll()
    sess = tui.ChatSession(tr, model="tiny", temperature=0.0, max_tokens=6)
    seen = []
    emit = lambda k, t: seen.append((k, t))
    ans = sess.ask("hello", emit)
    assert ans == "".join(t for k, t in seen if k == "content") and sess.messages[-1] == {"role": "assistant", "content": ans}
    assert sess.last_usage and sess.last_usage["completion_tokens"] == 6
    now[0] = 102.0
    dash.poll()
    s = dash.summary()
    assert s["arch"] == "dense_gqa" and s["decode_tok_s"] == 3.0 and s["error"] is None        # 6 tokens over 2 s
    assert s["ttft_p50_ms"] is not None and s["http_p50_ms"] is not None and s["free_blocks"] > 0
    con = Console(record=True, width=140)
    con.print(dash.render())
    out = con.export_text()
    assert "decode tok/s" in out and "TTFT p50" in out and "dense_gqa" in out
    # slash commands
    assert sess.command("/system be brief", emit) and sess.system == "be brief"
    assert sess.command("/thinking on", emit) and sess.thinking
    assert sess.command("/temp 0.3", emit) and sess.temperature == 0.3
    assert sess.command("/max 4", emit) and sess.max_tokens == 4
    assert sess.command("/temp x", emit) and sess.temperature == 0.3
    assert sess.command("/stats", emit) and "tok/s" in seen[-1][1]
    f = tmp_path / "conv.json"
    assert sess.command(f"/save {f}", emit) and len(json.loads(f.read_text())["messages"]) == 2
    sess.ask("again", emit)
    assert len(sess.messages) == 4
    assert sess.command("/clear", emit) and sess.messages == []
    assert sess.command("/bogus", emit) and "unknown command" in seen[-1][1]
    assert sess.command("/quit", emit) is False
    # scripted REPL: two inputs then EOF
    lines = iter(["/help", "hi"])

    def read(_prompt):
        try:
            return next(lines)
        except StopIteration:
            raise EOFError
    con2 = Console(record=True, width=100)
    tui.ChatSession(tr, model="tiny", max_tokens=3, temperature=0.0).repl(read, con2)
    assert "/thinking on|off" in con2.export_text()

    class Dead:
        def get_text(self, path):
            raise ConnectionError("refused")
    d2 = tui.Dashboard(Dead())
    d2.poll()
    assert "refused" in d2.summary()["error"]
    con.print(d2.render())


def test_http_sweep_against_a_real_listening_server():
    """uvicorn on a loopback port + the aiohttp SSE client of the benchmark: real sockets, real
    streaming, concurrent requests batched by the engine."""
    import socket
    import threading

    import uvicorn

    from metrale_inference_alpha_b200.bench.http_sweep import run_sweep
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=8, max_model_len=512))
    tok = load_tokenizer(None, eng.cfg.vocab_size)
    app = create_app(eng, tok, ServerConfig(model_name="tiny", auth_tokens=["k"]))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    try:
        end = time.time() + 20
        while not server.started and time.time() < end:
            time.sleep(0.05)
        assert server.started
        rows = run_sweep(f"http://127.0.0.1:{port}", [1, 4], isl_words=12, osl=5, model="tiny", api_key="k")
        assert [r["concurrency"] for r in rows] == [1, 4]
        for r in rows:
            assert r["errors"] == 0 and r["completion_tokens"] == 5 * r["concurrency"], r
            assert r["tok_s"] > 0 and r["ttft_p50_ms"] is not None and r["server_ttft_p50_ms"] is not None
        bad = run_sweep(f"http://127.0.0.1:{port}", [2], isl_words=4, osl=2, model="tiny", api_key="wrong")[0]
        assert bad["errors"] == 2 and "401" in bad["first_error"]
    finally:
        server.should_exit = True
        th.join(timeout=20)


def test_adaptive_sampling_rules_and_http_path():
    from metrale_inference_alpha_b200.sampling.adaptive import FREE, STRUCTURED, THINKING, TOOL_CALL, AdaptiveSampling
    a = AdaptiveSampling(0.0)
    assert a.temperature() == 0.0 and a.greedy(torch.zeros(8))                   # temperature 0 stays 0
    a = AdaptiveSampling(1.0, think_end_ids=[9], thinking_open=True, tool_open_ids=[5, 6], tool_close_ids=[7])
    assert a.update_zone([1, 2], False) == THINKING and a.temperature() == 1.0
    assert a.update_zone([1, 9, 2], False) == FREE
    assert a.update_zone([1, 9, 2], True) == STRUCTURED and abs(a.temperature() - 0.6) < 1e-9
    assert a.update_zone([1, 5, 6, 3], True) == TOOL_CALL and a.temperature() == 0.3   # capped; wins over grammar
    assert a.update_zone([1, 5, 6, 3, 7, 4], False) == THINKING                   # call closed, marker 9 not seen yet
    # greedy gate: thresholds per zone
    conf = torch.tensor([5.0, 0.0, 0.0, 0.0])                                     # top-1 = 0.98
    mid = torch.tensor([2.5, 0.0, 0.0, 0.0])                                      # top-1 = 0.80
    a.zone = FREE
    assert a.greedy(conf) and not a.greedy(mid)
    a.zone = TOOL_CALL
    assert a.greedy(mid)
    assert not a.greedy(torch.full((4,), float("-inf")))
    # entropy run: boosts after 8 / 16 / 32 confident tokens, reset by one uncertain token
    a = AdaptiveSampling(0.5)
    for n, want in ((7, 0.5), (1, 0.6), (8, 0.7), (16, 0.8)):
        for _ in range(n):
            a.observe(conf)
        assert abs(a.temperature() - want) < 1e-6, (n, a.temperature())
    a.observe(torch.zeros(16))
    assert a.low_entropy_run == 0 and a.temperature() == 0.5
    # repetition: a looping tail multiplies the temperature, varied output does not
    a.update_repetition([3, 4] * 40)
    assert a.lz_ratio < 0.15 and abs(a.temperature() - 0.9) < 1e-6
    b = AdaptiveSampling(0.5)
    b.update_repetition(list(range(1000, 1100)))
    assert b.lz_ratio > 0.35 and b.temperature() == 0.5
    b.update_repetition(list(range(1000, 1105)))                                  # fewer than 16 new tokens: not recomputed
    assert b._lz_checked_at == 100
    a.zone = TOOL_CALL
    assert a.temperature() == 0.3                                                 # no boost, no multiplier in a tool call
    # through the server: the flag attaches the state, seeded sampling stays reproducible
    from fastapi.testclient import TestClient
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=256))
    tok = load_tokenizer(None, eng.cfg.vocab_size)
    with TestClient(create_app(eng, tok, ServerConfig(model_name="tiny", adaptive_sampling=True))) as c:
        body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 12, "temperature": 0.9, "seed": 3,
                "return_token_ids": True}
        x = c.post("/v1/chat/completions", json=body).json()["choices"][0]["token_ids"]
        y = c.post("/v1/chat/completions", json=body).json()["choices"][0]["token_ids"]
        assert x == y and len(x) == 12
        z = c.post("/v1/chat/completions", json=dict(body, temperature=0)).json()["choices"][0]["token_ids"]
        assert len(z) == 12


def test_cross_turn_loop_detector():
    from metrale_inference_alpha_b200.server import loop_detector as LD
    call = lambda q: {"role": "assistant", "content": "Let me search the index for that file again to be sure.",
                      "tool_calls": [{"id": "c", "type": "function",
                                      "function": {"name": "search_files", "arguments": json.dumps({"query": q, "path": "/src", "limit": 20})}}]}
    tool = lambda text: {"role": "tool", "tool_call_id": "c", "content": text}
    user = {"role": "user", "content": "find the config loader"}
    assert LD.detect([LD.signature(call("a")), LD.signature(call("a"))]).kind == "none"        # fewer than 3 signatures
    same3 = [user, call("config loader"), tool("no results"), call("config loader"), tool("no results"),
             call("config loader"), tool("no results")]
    v = LD.check_loops(same3, tools_active=True)
    assert v.state.kind == "suppress" and v.state.run_length == 3 and v.state.score >= 0.65 and v.mask and v.bias == -4.0
    assert LD.check_loops(same3, tools_active=False).mask is False
    failing = [user] + [m for _ in range(3) for m in (call("config loader"), tool("Error: index not found"))]
    v = LD.check_loops(failing, True)
    assert v.state.kind == "suppress" and not v.mask and "failed" in v.reason
    moving = [user, call("config loader"), tool("3 results: a b c"), call("config loader"), tool("5 results: a b c d e"),
              call("config loader"), tool("9 results")]
    v = LD.check_loops(moving, True)
    assert v.state.kind == "suppress" and not v.mask and "change" in v.reason
    varied = [user, call("config loader"), tool("x"),
              {"role": "assistant", "content": "The loader lives in settings.py; I will open it and read the parse function now."},
              {"role": "assistant", "content": "Done: the function reads YAML first and falls back to environment variables when a key is missing."}]
    assert LD.check_loops(varied, True).state.kind == "none"
    os_env = __import__("os").environ
    os_env["METRALE_LOOP_NO_SUPPRESS"] = "1"
    try:
        assert LD.check_loops(same3, True).mask is False
    finally:
        del os_env["METRALE_LOOP_NO_SUPPRESS"]
    assert LD.jaccard(set(), {1}) == 0.0 and LD.jaccard({1, 2}, {2, 3}) == 1 / 3


def test_loop_detector_reaches_the_sampler_over_http(client):
    call = lambda: {"role": "assistant", "content": "search it again now ok go on pls",
                    "tool_calls": [{"id": "c", "type": "function", "function": {"name": "s", "arguments": json.dumps({"q": "x", "n": 2})}}]}
    msgs = [{"role": "user", "content": "find it"}]
    for _ in range(3):
        msgs += [call(), {"role": "tool", "tool_call_id": "c", "content": "none"}]
    tools = [{"type": "function", "function": {"name": "s", "parameters": {"type": "object"}}}]
    before = client.get("/metrics").text
    r = client.post("/v1/chat/completions", json={"messages": msgs, "tools": tools, "max_tokens": 4, "temperature": 0})
    assert r.status_code == 200
    after = client.get("/metrics").text
    assert "metrale_loop_suppress_total" in after and "metrale_loop_suppress_total" not in before


def test_n_choices_are_independent_samples(client):
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 1.2, "seed": 5, "n": 3,
            "return_token_ids": True}
    r = client.post("/v1/chat/completions", json=body).json()
    assert [c["index"] for c in r["choices"]] == [0, 1, 2]
    ids = [tuple(c["token_ids"]) for c in r["choices"]]
    assert all(len(i) == 6 for i in ids) and len(set(ids)) > 1                 # different seeds, different samples
    assert r["usage"]["completion_tokens"] == 18 and r["usage"]["total_tokens"] == r["usage"]["prompt_tokens"] + 18
    again = client.post("/v1/chat/completions", json=body).json()
    assert [tuple(c["token_ids"]) for c in again["choices"]] == ids             # reproducible per choice
    one = client.post("/v1/chat/completions", json=dict(body, n=1)).json()
    assert tuple(one["choices"][0]["token_ids"]) == ids[0]
    assert client.post("/v1/chat/completions", json=dict(body, n=2, stream=True)).status_code == 400
    assert client.post("/v1/chat/completions", json=dict(body, n=99)).status_code == 400


def test_prediction_field_reports_accepted_tokens(client):
    body = {"messages": [{"role": "user", "content": "say it"}], "max_tokens": 12, "temperature": 0, "return_token_ids": True}
    a = client.post("/v1/chat/completions", json=body).json()
    text = a["choices"][0]["message"]["content"] or ""
    tok = load_tokenizer(None, 4096)
    pred = tok.decode(a["choices"][0]["token_ids"], False) if hasattr(tok, "decode") else text
    b = client.post("/v1/chat/completions", json=dict(body, prediction={"type": "content", "content": pred})).json()
    assert b["choices"][0]["token_ids"] == a["choices"][0]["token_ids"]           # lossless
    det = b["usage"]["completion_tokens_details"]
    assert det["accepted_prediction_tokens"] + det["rejected_prediction_tokens"] >= 0
    if tok.encode(pred) == a["choices"][0]["token_ids"]:                           # the guess survived the text round trip
        assert det["accepted_prediction_tokens"] > 0


def test_guided_fields_map_onto_the_grammar_engine(client):
    from metrale_inference_alpha_b200.server.grammar import response_format_from_guided as rf
    assert rf({"guided_regex": "a+"}) == {"type": "regex", "pattern": "a+"}
    assert rf({"structured_outputs": {"json": {"type": "object"}}})["json_schema"]["schema"] == {"type": "object"}
    assert rf({"guided_json": '{"type": "integer"}'})["json_schema"]["schema"] == {"type": "integer"}
    assert rf({"guided_choice": ["yes", 'say "no"']})["grammar"] == 'root ::= "yes" | "say \\"no\\""'
    assert rf({"temperature": 0}) is None
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "pick"}], "max_tokens": 16,
                                                  "temperature": 0.7, "seed": 2, "guided_choice": ["alpha", "beta", "gamma delta"]}).json()
    assert r["choices"][0]["message"]["content"] in ("alpha", "beta", "gamma delta") and r["choices"][0]["finish_reason"] == "stop"
    r = client.post("/v1/completions", json={"prompt": "n=", "max_tokens": 8, "temperature": 0.8, "seed": 1,
                                              "guided_regex": r"[1-9]\d{2}"}).json()
    assert re.fullmatch(r"[1-9]\d{2}", r["choices"][0]["text"]) and r["choices"][0]["finish_reason"] == "stop"
    assert client.post("/v1/completions", json={"prompt": "x", "guided_regex": "(a"}).status_code == 400


def test_reasoning_effort_reaches_the_chat_template():
    from fastapi.testclient import TestClient
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=2, max_model_len=256))
    tok = load_tokenizer(None, eng.cfg.vocab_size)
    tok.chat_template = "{% for m in messages %}{{ m.content }}{% endfor %}|effort={{ reasoning_effort }}|"
    with TestClient(create_app(eng, tok, ServerConfig(model_name="tiny"))) as c:
        def n_prompt(**kw):
            r = c.post("/v1/chat/completions", json=dict({"messages": [{"role": "user", "content": "q"}], "max_tokens": 1}, **kw))
            assert r.status_code == 200, r.text
            return r.json()["usage"]["prompt_tokens"]
        base = len("q|effort=|")
        assert n_prompt() == base + len("none")                                           # thinking off
        assert n_prompt(enable_thinking=True) == base + len("medium")                     # on, nothing said
        assert n_prompt(enable_thinking=True, reasoning_effort="minimal") == base + len("minimal")
        assert n_prompt(enable_thinking=True, reasoning={"effort": "max"}) == base + len("max")
        assert n_prompt(reasoning_effort="high") == base + len("none")                    # ignored while thinking is off
        assert n_prompt(enable_thinking=True, chat_template_kwargs={"reasoning_effort": "low"}) == base + len("low")
        assert c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "q"}],
                                                    "reasoning_effort": "extreme"}).status_code == 400


def test_responses_api_streams_typed_events(client):
    with client.stream("POST", "/v1/responses", json={"input": "hello", "max_output_tokens": 5, "stream": True,
                                                       "temperature": 0}) as s:
        lines = [l for l in s.iter_lines() if l]
    kinds = [l[7:] for l in lines if l.startswith("event: ")]
    datas = [json.loads(l[6:]) for l in lines if l.startswith("data: ")]
    assert kinds[0] == "response.created" and kinds[-1] == "response.completed"
    assert kinds[1:3] == ["response.output_item.added", "response.content_part.added"]
    assert "response.output_text.done" in kinds and "response.output_item.done" in kinds
    assert [d["sequence_number"] for d in datas] == list(range(len(datas)))
    final = datas[-1]["response"]
    assert final["status"] == "completed" and final["usage"]["output_tokens"] == 5
    text = final["output"][-1]["content"][0]["text"]
    assert text == "".join(d["delta"] for d in datas if d["type"] == "response.output_text.delta")
    # the streamed response was stored: a follow-up continues it
    r = client.post("/v1/responses", json={"input": "more", "previous_response_id": final["id"], "max_output_tokens": 2}).json()
    assert r["status"] == "completed" and r["previous_response_id"] == final["id"]


def test_model_swap_keeps_the_listener_and_answers_with_the_new_model():
    """POST /v1/models/swap: the app, its routes and the scheduler thread stay; requests before the
    swap are answered by the old model, requests after it by the new one (a different preset gives
    different greedy tokens for the same prompt), and a bad model name leaves the old one serving."""
    from fastapi.testclient import TestClient
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    from metrale_inference_alpha_b200.server.tokenizer import load_tokenizer
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=128))
    tok = load_tokenizer(None, eng.cfg.vocab_size)
    body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 8, "temperature": 0, "return_token_ids": True}
    with TestClient(create_app(eng, tok, ServerConfig(model_name="m"))) as c:
        a = c.post("/v1/chat/completions", json=body).json()["choices"][0]["token_ids"]
        assert c.post("/v1/models/swap", json={"model": "no-such-model"}).status_code == 400
        assert c.post("/v1/chat/completions", json=body).json()["choices"][0]["token_ids"] == a
        r = c.post("/v1/models/swap", json={"model": "tiny-hybrid-moe", "served_model_name": "m2"})
        assert r.status_code == 200 and r.json()["swaps"] == 1 and r.json()["served_model_name"] == "m2"
        b = c.post("/v1/chat/completions", json=body).json()["choices"][0]["token_ids"]
        assert len(b) == 8 and b != a
        assert c.get("/serve-config").json()["model_config"]["arch"] == "qwen_hybrid"
        assert c.get("/health").status_code == 200
