"""HTTP surface: OpenAI ``/v1/chat/completions``, ``/v1/completions``, ``/v1/responses``,
``/v1/models``; Anthropic ``/v1/messages`` (+ ``/count_tokens``); ``/tokenize``, ``/health``,
``/health/live``, ``/metrics`` (Prometheus), ``/serve-config``, ``/memory``. SSE streaming,
usage blocks with the engine's timing extras, stop strings, logprobs, tool-call parsing,
reasoning split, JSON-constrained decoding, bearer auth, rate limiting, GPU-fault gate.
All three chat surfaces lower to one internal request (``_ChatJob``) like the reference's
shared IR (``crates/server/src/main_modules/serve_router.rs:44-141``, ``api/chat/mod.rs``,
``openai/chat_request.rs``, ``anthropic/types.rs``).
"""
from __future__ import annotations

import asyncio
import contextlib
import json
import os
import time
import uuid
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..sampling.params import SamplingParams
from ..utils.telemetry import Telemetry
from .chat_template import ChatRenderer
from .engine_loop import AsyncEngine
from .grammar import grammar_for_response_format, response_format_from_guided, tool_call_grammar
from .ratelimit import RateLimiter
from .reasoning_parser import ReasoningParser
from .conversation_store import ConversationStore
from .response_store import ResponseStore
from .tool_parser import StreamingToolDetector, parse_tool_calls


@dataclass
class ServerConfig:
    model_name: str = "model"
    auth_tokens: List[str] = field(default_factory=list)
    rate_per_s: float = 0.0
    tool_call_parser: str = "hermes"
    reasoning_format: str = "think"
    default_max_tokens: int = 1024
    tool_max_tokens: int = 8192
    request_timeout_s: float = 300.0
    telemetry: str = "basic"
    disable_thinking: bool = False
    default_top_n_sigma: float = 0.0    # sampling defaults for requests that do not set the field
    default_min_p: float = 0.0
    max_thinking_budget: int = 0        # cap (and default) of a request's thinking_token_budget; 0 = none
    content_loop_watchdog: float = 0.0  # > 0: LZ loop penalty applied when the request sets none
    loop_detector: bool = True          # cross-turn repetition: bias / mask the tool-call opener when an agent loops
    adaptive_sampling: bool = False     # per-token temperature by zone, confidence, entropy run and repetition
    dump_dir: str = ""                  # write every request / response pair as JSON files here
    otlp_endpoint: str = ""             # OTLP/HTTP collector (also METRALE_OTLP_ENDPOINT)
    tool_grammar: bool = False          # constrain tool calls with a grammar even under tool_choice "auto"


@dataclass
class _ChatJob:
    prompt_ids: List[int]
    params: SamplingParams
    tools: Optional[List[dict]] = None
    thinking_open: bool = False
    want_logprobs: bool = False
    return_token_ids: bool = False


def _sampling_from(body: Dict[str, Any], cfg: ServerConfig, max_key="max_tokens") -> SamplingParams:
    stop = body.get("stop") or body.get("stop_sequences") or []
    if isinstance(stop, str):
        stop = [stop]
    mt = body.get(max_key) or body.get("max_completion_tokens") or body.get("max_output_tokens")
    if mt is None:
        mt = cfg.tool_max_tokens if body.get("tools") else cfg.default_max_tokens
    return SamplingParams(
        max_tokens=int(mt), min_tokens=int(body.get("min_tokens") or 0),
        temperature=float(body.get("temperature", 1.0) if body.get("temperature") is not None else 1.0),
        top_k=int(body.get("top_k") or 0), top_p=float(body.get("top_p") or 1.0),
        min_p=float(body["min_p"] if body.get("min_p") is not None else cfg.default_min_p),
        top_n_sigma=float(body["top_n_sigma"] if body.get("top_n_sigma") is not None else cfg.default_top_n_sigma),
        repetition_penalty=float(body.get("repetition_penalty") or 1.0),
        presence_penalty=float(body.get("presence_penalty") or 0.0),
        frequency_penalty=float(body.get("frequency_penalty") or 0.0),
        dry_multiplier=float(body.get("dry_multiplier") or 0.0), dry_base=float(body.get("dry_base") or 1.75),
        dry_allowed_length=int(body.get("dry_allowed_length") or 2),
        lz_penalty=float((body.get("repetition_detection") or {}).get("penalty", 0.0)
                         if isinstance(body.get("repetition_detection"), dict) else cfg.content_loop_watchdog),
        logit_bias={int(k): float(v) for k, v in (body.get("logit_bias") or {}).items()},
        seed=body.get("seed"), stop=list(stop), logprobs=bool(body.get("logprobs")),
        top_logprobs=int(body.get("top_logprobs") or 0),
        timeout_s=float(body.get("timeout") or 0.0))


def create_app(engine, tokenizer, cfg: Optional[ServerConfig] = None, control=None) -> FastAPI:
    cfg = cfg or ServerConfig()
    # routes and the scheduler thread hold proxies, so `/v1/models/swap` can replace the engine (and
    # its tokenizer) behind a listener that stays up (server/model_swap.py)
    from .model_swap import Proxy
    engine = engine if isinstance(engine, Proxy) else Proxy(engine)
    tokenizer = tokenizer if isinstance(tokenizer, Proxy) else Proxy(tokenizer)
    aeng = AsyncEngine(engine, tokenizer, control)

    @contextlib.asynccontextmanager
    async def lifespan(_app):
        aeng.start()
        exporter = None
        endpoint = cfg.otlp_endpoint or os.environ.get("METRALE_OTLP_ENDPOINT", "")
        if endpoint and tel.enabled:
            from ..utils.otlp import OtlpExporter
            period = float(os.environ.get("METRALE_OTLP_PERIOD_S", "10"))
            exporter = OtlpExporter(tel, endpoint, period, gauges=lambda: {
                k: v for k, v in engine.stats().items() if isinstance(v, (int, float))}, service=cfg.model_name).start()
            _app.state.otlp = exporter
        yield
        aeng.shutdown(drain_s=15.0)        # drain in-flight requests, then stop the scheduler thread
        if exporter is not None:
            exporter.stop()

    app = FastAPI(title="metrale b200 engine", lifespan=lifespan)
    tel = Telemetry(cfg.telemetry)
    limiter = RateLimiter(cfg.rate_per_s)
    store = ResponseStore()
    conversations = ConversationStore()
    stored_completions: "OrderedDict[str, dict]" = OrderedDict()
    running_responses: Dict[str, Any] = {}
    renderer = ChatRenderer(getattr(tokenizer, "chat_template", None))
    app.state.engine, app.state.async_engine, app.state.telemetry = engine, aeng, tel
    eos = getattr(tokenizer, "eos_token_id", None)
    _close = {"think": "</think>", "mistral": "[/THINK]", "gemma4": "<channel|>"}.get(cfg.reasoning_format, "</think>")
    try:
        think_end_ids = list(tokenizer.encode(_close))
    except Exception:
        think_end_ids = []
    _opener = {"hermes": "<tool_call>", "qwen3": "<tool_call>", "qwen": "<tool_call>", "qwen3_xml": "<tool_call>",
               "qwen3_coder": "<tool_call>", "mistral": "[TOOL_CALLS]", "minimax_xml": "<minimax:tool_call>"}.get(cfg.tool_call_parser)
    try:
        tool_open_first = tokenizer.encode(_opener)[0] if _opener else None
    except Exception:
        tool_open_first = None
    engine.args.eos_token_id = engine.args.eos_token_id if engine.args.eos_token_id is not None else eos

    @app.middleware("http")
    async def gate(request: Request, call_next):
        t0 = time.perf_counter()
        path = request.url.path
        open_paths = ("/health", "/health/live", "/metrics")
        if path not in open_paths:
            if aeng.fatal or engine.fault.is_set():
                return JSONResponse({"error": {"message": aeng.fatal or engine.fault.reason(), "type": "gpu_fault"}}, 503)
            key = request.headers.get("authorization", "").removeprefix("Bearer ").strip() or \
                request.headers.get("x-api-key", "")
            if cfg.auth_tokens and key not in cfg.auth_tokens:
                return JSONResponse({"error": {"message": "invalid API key", "type": "authentication_error"}}, 401)
            if not limiter.allow(key or (request.client.host if request.client else "anon")):
                return JSONResponse({"error": {"message": "rate limit exceeded", "type": "rate_limit_error"}}, 429)
        limit = int(os.environ.get("METRALE_MAX_BODY_BYTES", "") or 32 << 20)
        clen = request.headers.get("content-length")
        if clen and clen.isdigit() and int(clen) > limit:
            return JSONResponse({"error": {"message": f"request body exceeds {limit} bytes", "type": "invalid_request_error"}}, 413)
        dump_body = None
        if cfg.dump_dir and request.method == "POST":
            dump_body = await request.body()         # cached by the request: the handler reads it again
        try:
            resp = await call_next(request)
        except Exception as e:                      # handler panic -> 500, server stays up
            tel.inc("http_500")
            return JSONResponse({"error": {"message": f"{type(e).__name__}: {e}", "type": "internal_error"}}, 500)
        tel.inc("http_requests")
        tel.observe_ms("http_latency", (time.perf_counter() - t0) * 1e3)
        if dump_body is not None:
            _dump_request(path, dump_body, resp.status_code, (time.perf_counter() - t0) * 1e3)
        return resp

    _dump_seq = [0]

    def _dump_request(path: str, body: bytes, status: int, ms: float) -> None:
        """One JSON file per POST: path, status, latency and the request body as sent."""
        try:
            os.makedirs(cfg.dump_dir, exist_ok=True)
            _dump_seq[0] += 1
            try:
                parsed = json.loads(body)
            except ValueError:
                parsed = body.decode("utf-8", "replace")
            name = f"{int(time.time() * 1e3):013d}-{_dump_seq[0]:06d}{path.replace('/', '_')}.json"
            with open(os.path.join(cfg.dump_dir, name), "w") as f:
                json.dump({"path": path, "status": status, "latency_ms": round(ms, 3), "request": parsed}, f)
        except OSError:
            tel.inc("dump_errors")

    # ------------------------------------------------------------------ plumbing
    def _job_from_chat(body: Dict[str, Any], messages, system=None, tools=None) -> _ChatJob:
        msgs = list(messages)
        choice = body.get("tool_choice")
        if choice == "none":
            tools = None
        elif isinstance(choice, dict) and tools:
            want = (choice.get("function") or {}).get("name") or choice.get("name")
            tools = [t for t in tools if t.get("function", {}).get("name") == want] or tools
        if system:
            msgs = [{"role": "system", "content": system}] + msgs
        thinking = body.get("enable_thinking")
        if thinking is None:
            th = body.get("thinking")
            thinking = bool(th and (th is True or th.get("type") == "enabled"))
        thinking = bool(thinking) and not cfg.disable_thinking
        kw = dict(body.get("chat_template_kwargs") or {})
        # the template variable `reasoning_effort`: the request's value (also as `reasoning.effort`)
        # while thinking is on, "medium" when it says nothing, "none" when thinking is off
        eff = body.get("reasoning_effort") or ((body.get("reasoning") or {}).get("effort") if isinstance(body.get("reasoning"), dict) else None)
        if eff is not None and eff not in ("none", "minimal", "low", "medium", "high", "max"):
            raise HTTPException(400, "reasoning_effort must be one of none, minimal, low, medium, high, max")
        kw.setdefault("reasoning_effort", (eff or "medium") if thinking else "none")
        text = renderer.render(msgs, tools=tools, add_generation_prompt=True, enable_thinking=thinking, **kw)
        ids = tokenizer.encode(text)
        sp = _sampling_from(body, cfg)
        from .chat_template import collect_images
        imgs = collect_images(msgs)
        if imgs:
            if getattr(engine, "vision", None) is None:
                raise HTTPException(400, "this model takes no image input")
            if any(not str(u).startswith("data:") for u in imgs):
                raise HTTPException(400, "images must be sent inline as data: URLs (the server fetches nothing)")
            sp.images = imgs
        if tools and cfg.loop_detector and tool_open_first is not None:
            from .loop_detector import check_loops
            verdict = check_loops(msgs, True)
            if verdict.state.kind != "none":
                tel.inc(f"loop_{verdict.state.kind}")
                sp.logit_bias = dict(sp.logit_bias)
                sp.logit_bias[tool_open_first] = -1e4 if verdict.mask else sp.logit_bias.get(tool_open_first, 0.0) + verdict.bias
        try:
            sp.grammar = grammar_for_response_format(body.get("response_format") or response_format_from_guided(body),
                                                     tokenizer, eos)
            forced = choice == "required" or (isinstance(choice, dict) and choice.get("type") not in ("auto", "none"))
            if sp.grammar is None and tools and (forced or cfg.tool_grammar) and hasattr(tokenizer, "token_bytes"):
                tg = tool_call_grammar(tools, cfg.tool_call_parser, "required" if forced else "auto")
                if tg is not None:
                    from ..grammar import TokenMatcher
                    sp.grammar = TokenMatcher(tg, tokenizer, eos)
        except ValueError as e:             # GrammarError: the schema / pattern / grammar does not compile
            raise HTTPException(400, f"invalid grammar: {e}")
        sp.adapter = body.get("adapter") or getattr(app.state, "active_adapter", None)
        pred = body.get("prediction")
        if isinstance(pred, dict) and pred.get("content"):
            pc = pred["content"]
            if isinstance(pc, list):
                pc = "".join(p_.get("text", "") for p_ in pc if isinstance(p_, dict))
            sp.prediction_ids = list(tokenizer.encode(pc))
        if cfg.adaptive_sampling and sp.temperature > 0:
            from ..sampling.adaptive import AdaptiveSampling
            opened = tokenizer.encode("<tool_call>") if tools and cfg.tool_call_parser in ("hermes", "qwen3", "qwen") else []
            closed = tokenizer.encode("</tool_call>") if opened else []
            sp.adaptive = AdaptiveSampling(sp.temperature, list(think_end_ids), bool(thinking), list(opened), list(closed))
        if thinking and think_end_ids:
            th = body.get("thinking") if isinstance(body.get("thinking"), dict) else {}
            want = body.get("thinking_token_budget") or th.get("budget_tokens") or 0
            budget = int(want or cfg.max_thinking_budget)
            if cfg.max_thinking_budget:
                budget = min(budget, cfg.max_thinking_budget)
            sp.thinking_budget, sp.think_end_ids = budget, list(think_end_ids)
        return _ChatJob(ids, sp, tools, thinking, bool(body.get("logprobs")), bool(body.get("return_token_ids")))

    def _account(usage) -> None:
        """Per-request telemetry from the usage block (what the dashboard and /metrics show)."""
        if not usage or not tel.enabled:
            return
        tel.inc("requests_finished")
        tel.inc("decode_tokens", float(usage.get("completion_tokens") or 0))
        tel.inc("prefill_tokens", float(usage.get("prompt_tokens") or 0))
        if usage.get("time_to_first_token_ms") is not None:
            tel.observe_ms("ttft", float(usage["time_to_first_token_ms"]))

    async def _collect(job: _ChatJob):
        text, ids, usage, reason, lps = "", [], None, None, None
        async for ev in aeng.submit(job.prompt_ids, job.params):
            if ev.error:
                raise HTTPException(500 if "fault" in (ev.error or "") else 400, ev.error)
            text += ev.text
            ids += ev.token_ids
            if ev.finished:
                usage, reason, lps = ev.usage, ev.finish_reason, ev.logprobs
                _account(usage)
        return text, ids, usage, reason, lps

    def _split_outputs(job: _ChatJob, text: str):
        rp = ReasoningParser(cfg.reasoning_format, starts_open=job.thinking_open)
        r, c = rp.push(text)
        r2, c2 = rp.flush()
        reasoning, content = r + r2, c + c2
        calls = []
        if job.tools:
            content, calls = parse_tool_calls(content, cfg.tool_call_parser, job.tools)
        return reasoning, content, calls

    def _lp_block(ids, lps):
        if not lps:
            return None
        return {"content": [{"token": tokenizer.decode([t], False), "logprob": lp, "bytes": None, "top_logprobs": []}
                            for t, lp in zip(ids, lps)]}

    # ------------------------------------------------------------------ OpenAI
    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": cfg.model_name, "object": "model", "owned_by": "metrale-b200",
                                            "max_model_len": engine.sched_cfg.max_model_len}]}

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        body = await request.json()
        if not body.get("messages"):
            raise HTTPException(400, "messages is required")
        n = int(body.get("n") or 1)
        if n < 1 or n > 16:
            raise HTTPException(400, "n must be between 1 and 16")
        if n > 1 and body.get("stream"):
            raise HTTPException(400, "n > 1 is supported for non-streaming requests")
        job = _job_from_chat(body, body["messages"], tools=body.get("tools"))
        rid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        if not body.get("stream"):
            # n choices = n independent samples of the same prompt (the prefix cache shares its KV);
            # a seeded request gives choice i the seed + i
            jobs = [job]
            for i in range(1, n):
                b_i = dict(body, seed=body["seed"] + i) if body.get("seed") is not None else body
                jobs.append(_job_from_chat(b_i, body["messages"], tools=body.get("tools")))
            results = await asyncio.gather(*(_collect(j) for j in jobs))
            choices, usage = [], None
            for i, (j, (text, ids, u, reason, lps)) in enumerate(zip(jobs, results)):
                reasoning, content, calls = _split_outputs(j, text)
                msg: Dict[str, Any] = {"role": "assistant", "content": content or (None if calls else "")}
                if reasoning:
                    msg["reasoning_content"] = reasoning
                if calls:
                    msg["tool_calls"] = calls
                    reason = "tool_calls"
                choice = {"index": i, "message": msg, "finish_reason": reason, "logprobs": _lp_block(ids, lps)}
                if j.return_token_ids:
                    choice["token_ids"] = ids
                choices.append(choice)
                if usage is None:
                    usage = dict(u or {})
                elif u:
                    usage["completion_tokens"] = (usage.get("completion_tokens") or 0) + (u.get("completion_tokens") or 0)
                    usage["total_tokens"] = (usage.get("prompt_tokens") or 0) + usage["completion_tokens"]
            out = {"id": rid, "object": "chat.completion", "created": created, "model": cfg.model_name,
                   "choices": choices, "usage": usage}
            if body.get("store"):
                stored_completions[rid] = dict(out, metadata=body.get("metadata") or {})
                while len(stored_completions) > 1024:
                    stored_completions.popitem(last=False)
            return out

        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

        async def gen():
            def chunk(delta, finish=None, usage=None):
                d = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": cfg.model_name,
                     "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
                if usage is not None:
                    d["usage"] = usage
                return f"data: {json.dumps(d)}\n\n"
            yield chunk({"role": "assistant", "content": ""})
            rp = ReasoningParser(cfg.reasoning_format, starts_open=job.thinking_open)
            td = StreamingToolDetector() if job.tools else None
            final_usage, reason = None, None
            async for ev in aeng.submit(job.prompt_ids, job.params):
                if ev.error:
                    yield f"data: {json.dumps({'error': {'message': ev.error}})}\n\n"
                    break
                r, c = rp.push(ev.text)
                if ev.finished:
                    r2, c2 = rp.flush()
                    r, c = r + r2, c + c2
                if td is not None:
                    c = td.push(c)
                if r:
                    yield chunk({"reasoning_content": r})
                if c:
                    yield chunk({"content": c})
                if ev.finished:
                    final_usage, reason = ev.usage, ev.finish_reason
                    _account(final_usage)
            if td is not None:
                held = td.finish()
                if held:
                    rest, calls = parse_tool_calls(held, cfg.tool_call_parser, job.tools)
                    if rest:
                        yield chunk({"content": rest})
                    for i, cl in enumerate(calls):
                        yield chunk({"tool_calls": [dict(cl, index=i)]})
                    if calls:
                        reason = "tool_calls"
            yield chunk({}, finish=reason or "stop")
            if include_usage and final_usage:
                d = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": cfg.model_name,
                     "choices": [], "usage": final_usage}
                yield f"data: {json.dumps(d)}\n\n"
            yield "data: [DONE]\n\n"
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await request.json()
        prompt = body.get("prompt")
        if prompt is None:
            raise HTTPException(400, "prompt is required")
        ids = prompt if (isinstance(prompt, list) and prompt and isinstance(prompt[0], int)) else \
            tokenizer.encode(prompt if isinstance(prompt, str) else prompt[0])
        sp = _sampling_from(body, cfg)
        sp.adapter = body.get("adapter")
        if body.get("ignore_eos"):
            sp.ignore_eos = True
        try:
            sp.grammar = grammar_for_response_format(body.get("response_format") or response_format_from_guided(body),
                                                     tokenizer, eos)
        except ValueError as e:
            raise HTTPException(400, f"invalid grammar: {e}")
        job = _ChatJob(ids, sp)
        rid, created = "cmpl-" + uuid.uuid4().hex[:24], int(time.time())
        if not body.get("stream"):
            text, out_ids, usage, reason, lps = await _collect(job)
            ch = {"index": 0, "text": text, "finish_reason": reason, "logprobs": None}
            if body.get("return_token_ids"):
                ch["token_ids"] = out_ids
            if lps:
                ch["logprobs"] = {"token_logprobs": lps, "tokens": [tokenizer.decode([t], False) for t in out_ids]}
            return {"id": rid, "object": "text_completion", "created": created, "model": cfg.model_name,
                    "choices": [ch], "usage": usage}

        async def gen():
            usage = None
            async for ev in aeng.submit(job.prompt_ids, job.params):
                if ev.error:
                    yield f"data: {json.dumps({'error': {'message': ev.error}})}\n\n"
                    break
                d = {"id": rid, "object": "text_completion", "created": created, "model": cfg.model_name,
                     "choices": [{"index": 0, "text": ev.text, "finish_reason": ev.finish_reason if ev.finished else None}]}
                if ev.finished:
                    d["usage"] = ev.usage
                    _account(ev.usage)
                yield f"data: {json.dumps(d)}\n\n"
            yield "data: [DONE]\n\n"
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.get("/v1/responses/{response_id}")
    async def get_response(response_id: str):
        r = store.get(response_id)
        if r is None:
            raise HTTPException(404, "unknown response id")
        return {"id": response_id, "object": "response", "status": "completed", "previous_response_id": r["previous"],
                "output": [{"type": "message", "role": "assistant",
                            "content": [{"type": "output_text", "text": r["output"], "annotations": []}]}]}

    @app.delete("/v1/responses/{response_id}")
    async def delete_response(response_id: str):
        if not store.delete(response_id):
            raise HTTPException(404, "unknown response id")
        return {"id": response_id, "object": "response.deleted", "deleted": True}

    @app.get("/v1/responses/{response_id}/input_items")
    async def response_input_items(response_id: str):
        r = store.get(response_id)
        if r is None:
            raise HTTPException(404, "unknown response id")
        data = [{"type": "message", "id": f"msg_{response_id[5:]}_{i}", "role": m.get("role", "user"),
                 "content": [{"type": "input_text", "text": m.get("content") if isinstance(m.get("content"), str) else ""}]}
                for i, m in enumerate(r["messages"])]
        return {"object": "list", "data": data, "first_id": data[0]["id"] if data else None,
                "last_id": data[-1]["id"] if data else None, "has_more": False}

    @app.post("/v1/responses/{response_id}/cancel")
    async def cancel_response(response_id: str):
        t = running_responses.get(response_id)
        if t is None:
            if store.get(response_id) is not None:
                raise HTTPException(400, "the response has already completed")
            raise HTTPException(404, "unknown response id")
        t.cancel()
        return {"id": response_id, "object": "response", "status": "cancelled"}

    async def _responses_stream(body, job, rid, new_msgs, prev, conv_id):
        """Responses API event stream: response.created, output_item.added, content_part.added,
        output_text.delta ..., output_text.done, output_item.done, response.completed (with usage)."""
        seq = [0]

        def ev(kind: str, **fields) -> str:
            d = {"type": kind, "sequence_number": seq[0], **fields}
            seq[0] += 1
            return f"event: {kind}\ndata: {json.dumps(d)}\n\n"
        shell = {"id": rid, "object": "response", "created_at": int(time.time()), "model": cfg.model_name,
                 "previous_response_id": prev, "status": "in_progress", "output": []}
        yield ev("response.created", response=shell)
        mid = "msg_" + uuid.uuid4().hex[:16]
        item = {"type": "message", "id": mid, "role": "assistant", "status": "in_progress", "content": []}
        yield ev("response.output_item.added", output_index=0, item=item)
        yield ev("response.content_part.added", item_id=mid, output_index=0, content_index=0,
                 part={"type": "output_text", "text": "", "annotations": []})
        rp = ReasoningParser(cfg.reasoning_format, starts_open=job.thinking_open)
        text, reasoning, usage, status = "", "", None, "completed"
        async for e in aeng.submit(job.prompt_ids, job.params):
            if e.error:
                status = "failed"
                yield ev("error", message=e.error)
                break
            r, c = rp.push(e.text)
            if e.finished:
                r2, c2 = rp.flush()
                r, c = r + r2, c + c2
                usage = e.usage
                _account(usage)
            reasoning += r
            if c:
                text += c
                yield ev("response.output_text.delta", item_id=mid, output_index=0, content_index=0, delta=c)
        content, calls = (parse_tool_calls(text, cfg.tool_call_parser, job.tools) if job.tools else (text, []))
        yield ev("response.output_text.done", item_id=mid, output_index=0, content_index=0, text=content)
        done_item = dict(item, status="completed", content=[{"type": "output_text", "text": content, "annotations": []}])
        yield ev("response.output_item.done", output_index=0, item=done_item)
        out = ([{"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:16], "summary": [{"type": "summary_text", "text": reasoning}]}]
               if reasoning else []) + [done_item]
        for cl in calls:
            out.append({"type": "function_call", "call_id": cl["id"], "name": cl["function"]["name"],
                        "arguments": cl["function"]["arguments"]})
        u = usage or {}
        if status == "completed" and body.get("store", True):
            store.put(rid, new_msgs, content, prev)
        if status == "completed" and conv_id:
            items = [dict(m, type="message") for m in new_msgs if isinstance(m.get("content"), str)]
            items.append({"type": "message", "role": "assistant", "content": content})
            try:
                conversations.add_items(conv_id, items[-20:])
            except (KeyError, ValueError):
                pass
        yield ev("response.completed" if status == "completed" else "response.failed",
                 response=dict(shell, status=status, output=out,
                               usage={"input_tokens": u.get("prompt_tokens"), "output_tokens": u.get("completion_tokens"),
                                      "total_tokens": u.get("total_tokens")}))

    @app.post("/v1/responses")
    async def responses(request: Request):
        body = await request.json()
        inp = body.get("input")
        new_msgs = [{"role": "user", "content": inp}] if isinstance(inp, str) else [
            {"role": m.get("role", "user"), "content": m.get("content")} for m in (inp or [])]
        prev = body.get("previous_response_id")
        history = []
        if prev:
            try:
                history = store.thread(prev)
            except KeyError:
                raise HTTPException(404, f"unknown previous_response_id {prev!r}")
        conv = body.get("conversation")
        conv_id = conv.get("id") if isinstance(conv, dict) else conv
        if conv_id:
            if prev:
                raise HTTPException(400, "`conversation` and `previous_response_id` are mutually exclusive")
            try:
                history = conversations.messages(conv_id)
            except KeyError:
                raise HTTPException(404, f"unknown conversation {conv_id!r}")
        messages = history + new_msgs
        job = _job_from_chat(body, messages, system=body.get("instructions"), tools=body.get("tools"))
        rid = "resp_" + uuid.uuid4().hex[:24]
        if body.get("stream"):
            return StreamingResponse(_responses_stream(body, job, rid, new_msgs, prev, conv_id), media_type="text/event-stream")
        task = asyncio.ensure_future(_collect(job))
        running_responses[rid] = task
        try:
            text, ids, usage, reason, _ = await task
        except asyncio.CancelledError:
            return {"id": rid, "object": "response", "status": "cancelled", "model": cfg.model_name, "output": []}
        finally:
            running_responses.pop(rid, None)
        reasoning, content, calls = _split_outputs(job, text)
        out = []
        if reasoning:
            out.append({"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:16], "summary": [{"type": "summary_text", "text": reasoning}]})
        out.append({"type": "message", "id": "msg_" + uuid.uuid4().hex[:16], "role": "assistant", "status": "completed",
                    "content": [{"type": "output_text", "text": content, "annotations": []}]})
        for c in calls:
            out.append({"type": "function_call", "call_id": c["id"], "name": c["function"]["name"],
                        "arguments": c["function"]["arguments"]})
        u = usage or {}
        if body.get("store", True):
            store.put(rid, new_msgs, content, prev)
        if conv_id:
            items = [dict(m, type="message") for m in new_msgs if isinstance(m.get("content"), str)]
            items.append({"type": "message", "role": "assistant", "content": content})
            try:
                conversations.add_items(conv_id, items[-20:])
            except (KeyError, ValueError):
                pass                           # deleted or full meanwhile: the response itself stands
        return {"id": rid, "object": "response", "created_at": int(time.time()), "previous_response_id": prev,
                "model": cfg.model_name, "status": "completed", "output": out,
                "usage": {"input_tokens": u.get("prompt_tokens"), "output_tokens": u.get("completion_tokens"),
                          "total_tokens": u.get("total_tokens")}}

    # ------------------------------------------------------------------ Anthropic
    @app.post("/v1/messages")
    async def messages(request: Request):
        body = await request.json()
        if "max_tokens" not in body:
            raise HTTPException(400, "max_tokens is required")
        tools = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                                   "parameters": t.get("input_schema", {})}} for t in body.get("tools", [])] or None
        job = _job_from_chat(body, body.get("messages", []), system=body.get("system"), tools=tools)
        mid = "msg_" + uuid.uuid4().hex[:24]

        def blocks(reasoning, content, calls):
            out = []
            if reasoning:
                out.append({"type": "thinking", "thinking": reasoning})
            if content:
                out.append({"type": "text", "text": content})
            for c in calls:
                out.append({"type": "tool_use", "id": c["id"].replace("call_", "toolu_"), "name": c["function"]["name"],
                            "input": json.loads(c["function"]["arguments"] or "{}")})
            return out
        stop_map = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use"}
        if not body.get("stream"):
            text, ids, usage, reason, _ = await _collect(job)
            reasoning, content, calls = _split_outputs(job, text)
            u = usage or {}
            hit = None
            if reason == "stop" and job.params.stop:
                reason, hit = "stop_sequence", None
            return {"id": mid, "type": "message", "role": "assistant", "model": cfg.model_name,
                    "content": blocks(reasoning, content, calls),
                    "stop_reason": "tool_use" if calls else (reason if reason == "stop_sequence" else stop_map.get(reason, reason)),
                    "stop_sequence": hit,
                    "usage": {"input_tokens": u.get("prompt_tokens"), "output_tokens": u.get("completion_tokens"),
                              "cache_read_input_tokens": (u.get("prompt_tokens_details") or {}).get("cached_tokens", 0)}}

        async def gen():
            def sse(ev, data):
                return f"event: {ev}\ndata: {json.dumps(data)}\n\n"
            yield sse("message_start", {"type": "message_start", "message": {
                "id": mid, "type": "message", "role": "assistant", "model": cfg.model_name, "content": [],
                "stop_reason": None, "usage": {"input_tokens": len(job.prompt_ids), "output_tokens": 0}}})
            yield sse("content_block_start", {"type": "content_block_start", "index": 0,
                                              "content_block": {"type": "text", "text": ""}})
            usage, reason = None, None
            async for ev in aeng.submit(job.prompt_ids, job.params):
                if ev.text:
                    yield sse("content_block_delta", {"type": "content_block_delta", "index": 0,
                                                      "delta": {"type": "text_delta", "text": ev.text}})
                if ev.finished:
                    usage, reason = ev.usage, ev.finish_reason
                    _account(usage)
            yield sse("content_block_stop", {"type": "content_block_stop", "index": 0})
            yield sse("message_delta", {"type": "message_delta",
                                        "delta": {"stop_reason": stop_map.get(reason, reason), "stop_sequence": None},
                                        "usage": {"output_tokens": (usage or {}).get("completion_tokens", 0)}})
            yield sse("message_stop", {"type": "message_stop"})
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(request: Request):
        body = await request.json()
        job = _job_from_chat({"max_tokens": 1}, body.get("messages", []), system=body.get("system"))
        return {"input_tokens": len(job.prompt_ids)}

    # ------------------------------------------------------------------ utility routes
    @app.post("/tokenize")
    async def tokenize(request: Request):
        body = await request.json()
        ids = tokenizer.encode(body.get("prompt") or body.get("text") or "")
        return {"tokens": ids, "count": len(ids), "max_model_len": engine.sched_cfg.max_model_len}

    @app.post("/detokenize")
    async def detokenize(request: Request):
        body = await request.json()
        return {"prompt": tokenizer.decode(body.get("tokens", []))}

    @app.get("/health")
    async def health():
        if aeng.fatal or engine.fault.is_set():
            return JSONResponse({"status": "gpu_fault", "reason": aeng.fatal or engine.fault.reason()}, 503)
        return {"status": "ok"}

    @app.get("/health/live")
    async def live():
        return {"status": "alive"}

    @app.get("/metrics")
    async def metrics():
        st = engine.stats()
        flat = {f"engine_{k}": v for k, v in st.items() if isinstance(v, (int, float))}
        return PlainTextResponse(tel.prometheus(flat))

    @app.get("/serve-config")
    async def serve_config():
        a = engine.args
        return {"model": cfg.model_name, "engine": {k: (v if isinstance(v, (int, float, str, bool, type(None))) else str(v))
                                                     for k, v in vars(a).items()},
                "model_config": json.loads(engine.cfg.to_json())}

    @app.get("/memory")
    async def memory():
        st = engine.stats()
        return {"weights_bytes": st.get("weights_bytes"), "kv_bytes": engine.runner.kv_bytes(),
                "kv_blocks": st.get("kv_blocks"), "free_blocks": st.get("free_blocks")}

    from .extra_routes import install as _install_extra
    _install_extra(app, engine=engine, tokenizer=tokenizer, cfg=cfg, telemetry=tel, conversations=conversations,
                   completions=stored_completions)
    return app
