"""Routes beside the generation endpoints: conversations, stored chat completions, LoRA slot
control, model lookup, introspection (``/hardware``, ``/forward``, ``/v1/events``) and the OpenAI
endpoints this engine does not serve, which answer 501 with an OpenAI-shaped error instead of 404.

Role of the reference's ``crates/server/src/api/{conversations,stubs,misc_handlers,
telemetry_events,lora}.rs`` as routed by ``main_modules/serve_router.rs``.
"""
from __future__ import annotations

import asyncio
import functools
import json
import time
from typing import Any, Dict, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

from .conversation_store import ConversationError, ConversationStore


def openai_error(status: int, message: str, param: Optional[str] = None, code: Optional[str] = None,
                 etype: Optional[str] = None) -> JSONResponse:
    kind = etype or {400: "invalid_request_error", 404: "not_found_error", 501: "not_implemented_error"}.get(status, "api_error")
    return JSONResponse({"error": {"message": message, "type": kind, "param": param, "code": code}}, status)


_STUBS = {
    "embeddings": (["POST /v1/embeddings"],
                   "Embeddings are not supported by this model: the engine serves generative (chat / completion) models only."),
    "batches": (["POST /v1/batches", "GET /v1/batches", "GET /v1/batches/{id}", "DELETE /v1/batches/{id}",
                 "POST /v1/batches/{id}/cancel"], "The Batch API is not implemented: send requests to /v1/chat/completions directly."),
    "files": (["POST /v1/files", "GET /v1/files", "GET /v1/files/{id}", "DELETE /v1/files/{id}", "GET /v1/files/{id}/content"],
              "The Files API is not implemented."),
    "audio": (["POST /v1/audio/transcriptions", "POST /v1/audio/translations", "POST /v1/audio/speech"],
              "Audio endpoints are not implemented: the engine serves text generation only."),
    "images": (["POST /v1/images/generations", "POST /v1/images/edits", "POST /v1/images/variations"],
               "Image endpoints are not implemented: the engine serves text generation only."),
    "moderations": (["POST /v1/moderations"], "The Moderations API is not implemented."),
}


def install(app: FastAPI, *, engine, tokenizer, cfg, telemetry, conversations: ConversationStore,
            completions: Dict[str, dict], events_period_s: float = 1.0) -> None:
    # ------------------------------------------------------------------ 501 stubs
    for _, (routes, message) in _STUBS.items():
        for r in routes:
            method, path = r.split(" ")

            async def stub(request: Request, _m=message):
                return openai_error(501, _m, code="not_implemented")
            app.add_api_route(path, stub, methods=[method])

    # ------------------------------------------------------------------ conversations
    def guarded(fn):
        @functools.wraps(fn)               # FastAPI reads the handler's signature through __wrapped__
        async def run(*a, **kw):
            try:
                return await fn(*a, **kw)
            except ConversationError as e:
                return openai_error(400, str(e), e.param, e.code)
            except KeyError as e:
                return openai_error(404, f"not found: {e.args[0]}", code="not_found")
        return run

    async def _body(request: Request) -> dict:
        try:
            b = await request.json()
            return b if isinstance(b, dict) else {}
        except ValueError:
            return {}

    @app.post("/v1/conversations")
    @guarded
    async def create_conversation(request: Request):
        b = await _body(request)
        return ConversationStore.public(conversations.create(b.get("items"), b.get("metadata")))

    @app.get("/v1/conversations/{cid}")
    @guarded
    async def get_conversation(cid: str):
        return ConversationStore.public(conversations.get(cid))

    @app.post("/v1/conversations/{cid}")
    @guarded
    async def update_conversation(cid: str, request: Request):
        return ConversationStore.public(conversations.update(cid, (await _body(request)).get("metadata")))

    @app.delete("/v1/conversations/{cid}")
    @guarded
    async def delete_conversation(cid: str):
        if not conversations.delete(cid):
            raise KeyError(cid)
        return {"id": cid, "object": "conversation.deleted", "deleted": True}

    @app.post("/v1/conversations/{cid}/items")
    @guarded
    async def add_items(cid: str, request: Request):
        items = (await _body(request)).get("items")
        if not isinstance(items, list) or not items:
            raise ConversationError("`items` must be a non-empty array", "items", "items_missing")
        new = conversations.add_items(cid, items)
        return {"object": "list", "data": new, "first_id": new[0]["id"], "last_id": new[-1]["id"], "has_more": False}

    @app.get("/v1/conversations/{cid}/items")
    @guarded
    async def list_items(cid: str, limit: int = 20, after: Optional[str] = None, order: str = "desc"):
        return conversations.list_items(cid, limit, after, order)

    @app.get("/v1/conversations/{cid}/items/{item_id}")
    @guarded
    async def get_item(cid: str, item_id: str):
        return conversations.get_item(cid, item_id)

    @app.delete("/v1/conversations/{cid}/items/{item_id}")
    @guarded
    async def delete_item(cid: str, item_id: str):
        return ConversationStore.public(conversations.delete_item(cid, item_id))

    # ------------------------------------------------------------------ stored chat completions
    @app.get("/v1/chat/completions/{completion_id}")
    async def get_stored_completion(completion_id: str):
        r = completions.get(completion_id)
        if r is None:
            return openai_error(404, f"no stored completion {completion_id!r} (send `store: true` to keep one)", code="not_found")
        return r

    # ------------------------------------------------------------------ models / LoRA
    @app.get("/v1/models/{model_id:path}")
    async def get_model(model_id: str):
        names = {cfg.model_name} | set(getattr(getattr(engine.runner.decoder, "lora", None), "names", lambda: [])())
        if model_id not in names:
            return openai_error(404, f"The model '{model_id}' does not exist", "model", "model_not_found")
        return {"id": model_id, "object": "model", "owned_by": "metrale-b200", "max_model_len": engine.sched_cfg.max_model_len}

    @app.post("/v1/models/swap")
    async def model_swap(request: Request):
        """Load another model (preset name or checkpoint directory) behind the running listener.
        In-flight requests finish on the old model, later ones are answered by the new one."""
        b = await _body(request)
        model = b.get("model")
        if not model:
            return openai_error(400, "`model` is required", "model")
        aeng = app.state.async_engine
        if aeng.control is not None:
            return openai_error(501, "model swap is not available on a multi-rank engine", code="not_implemented")
        from .model_swap import build_like
        try:
            new = await asyncio.get_running_loop().run_in_executor(
                None, lambda: aeng.request_swap(lambda: build_like(engine.target(), model, b.get("tokenizer"))))
        except (OSError, ValueError, KeyError, RuntimeError, TimeoutError) as e:
            return openai_error(400, f"cannot load model: {e}", "model", "model_swap_failed")
        if b.get("served_model_name"):
            cfg.model_name = b["served_model_name"]
        return {"status": "swapped", "model": new.cfg.name, "served_model_name": cfg.model_name, "swaps": engine.swaps}

    @app.post("/v1/lora/load")
    async def lora_load(request: Request):
        b = await _body(request)
        name, path = b.get("name") or b.get("lora_name"), b.get("path") or b.get("lora_path")
        if not name or not path:
            return openai_error(400, "`name` and `path` are required", "name")
        try:
            await asyncio.get_running_loop().run_in_executor(
                None, lambda: engine.load_adapter(name, path, int(b.get("max_loras", 8)), int(b.get("max_rank", 16))))
        except (OSError, ValueError, KeyError) as e:
            return openai_error(400, f"cannot load adapter: {e}", "path", "lora_load_failed")
        return {"status": "loaded", "name": name}

    @app.post("/v1/lora/active")
    async def lora_active(request: Request):
        b = await _body(request)
        name = b.get("name")
        lora = getattr(engine.runner.decoder, "lora", None)
        known = set(lora.names()) if lora is not None and hasattr(lora, "names") else set()
        if name is not None and name not in known:
            return openai_error(404, f"adapter {name!r} is not loaded", "name", "lora_not_found")
        app.state.active_adapter = name            # requests without an `adapter` field follow it
        return {"active": name}

    # ------------------------------------------------------------------ introspection
    @app.get("/hardware")
    async def hardware():
        from .cli import doctor
        rep = await asyncio.get_running_loop().run_in_executor(None, doctor)
        return {k: rep.get(k) for k in ("devices", "cuda_available", "cuda_runtime", "torch", "nccl", "p2p", "native_library")}

    @app.get("/forward")
    async def forward():
        import os
        a, c = engine.args, engine.cfg
        return {"model": cfg.model_name, "arch": c.arch, "layers": c.num_layers, "weight_format": c.weight_format,
                "kv_dtype": c.kv_dtype, "block_size": a.block_size, "max_num_seqs": a.max_num_seqs,
                "max_model_len": engine.sched_cfg.max_model_len, "cuda_graphs": bool(engine.runner.use_graphs),
                "speculative": engine.spec_mode, "num_drafts": a.num_drafts, "tp_size": engine.tp.size, "ep_size": a.ep_size,
                "fused_collectives": a.fused_collectives, "static_act_scales": bool(getattr(engine, "calibrated_layers", 0)),
                "pdl": os.environ.get("METRALE_PDL", "2"), "device": str(engine.device)}

    @app.get("/v1/events")
    async def events(request: Request, limit: int = 0):
        if not telemetry.enabled:
            return openai_error(404, "telemetry is off: start the server with --telemetry basic (or kernel) to stream /v1/events")

        async def gen():
            seq = 0
            while not await request.is_disconnected():
                snap = {"seq": seq, "at": time.time(), "counters": dict(telemetry.counters), "gauges": dict(telemetry.gauges),
                        "engine": {k: v for k, v in engine.stats().items() if isinstance(v, (int, float))}}
                yield f"data: {json.dumps(snap)}\n\n"
                seq += 1
                if limit and seq >= limit:
                    return
                await asyncio.sleep(events_period_s)
        return StreamingResponse(gen(), media_type="text/event-stream")
