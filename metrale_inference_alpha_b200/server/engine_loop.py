"""Bridges the synchronous engine (one scheduler thread that owns the CUDA context) and the
asyncio HTTP handlers: requests go in through a thread-safe queue, token events come back on
per-request asyncio queues. Handles stop strings (with hold-back so a partial match is never
streamed), incremental detokenisation and client-disconnect aborts.
Role of the reference's scheduler OS thread + ``mpsc<InferenceRequest>`` / ``StreamEvent``
channels (``crates/server/src/api/inference_types.rs:61-264``)."""
from __future__ import annotations

import asyncio
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..sampling.params import SamplingParams
from .tokenizer import IncrementalDetokenizer


@dataclass
class StreamEvent:
    text: str = ""
    token_ids: List[int] = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[str] = None
    usage: Optional[dict] = None
    logprobs: Optional[List[float]] = None
    error: Optional[str] = None


class _Live:
    def __init__(self, loop, detok, stops: List[str]):
        self.q: asyncio.Queue = asyncio.Queue()
        self.loop = loop
        self.detok = detok
        self.stops = stops
        self.held = ""
        self.text_len = 0
        self.t0 = time.time()
        self.t_first: Optional[float] = None


class AsyncEngine:
    def __init__(self, engine, tokenizer, control=None):
        """``control``: a ``parallel.control.ControlPlane`` when this is rank 0 of a multi-rank
        engine; every tick's operations are published to the follower ranks before they are
        applied here, so all schedulers stay in lockstep."""
        self.engine, self.tokenizer, self.control = engine, tokenizer, control
        self._in: "queue.Queue" = queue.Queue()
        self._live: Dict[str, _Live] = {}
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="scheduler", daemon=True)
        self.fatal: Optional[str] = None

    def start(self) -> None:
        self._thread.start()

    def shutdown(self, drain_s: float = 15.0) -> None:
        t0 = time.time()
        while self._live and time.time() - t0 < drain_s:
            time.sleep(0.05)
        self._stop.set()
        self._thread.join(timeout=5)
        close = getattr(self.engine, "close", None)
        if close is not None and not self._thread.is_alive():      # the scheduler thread is gone: tear the engine down in order
            try:
                close()
            except Exception:
                pass
        if self.control is not None and not self.fatal:
            try:
                self.control.exchange([("shutdown", None, None, None)])
                self.control.leave()
            except Exception:
                pass

    # ---- called from handlers (event loop thread)
    async def submit(self, prompt_ids: List[int], params: SamplingParams, request_id: Optional[str] = None):
        """Async generator of StreamEvent for one request."""
        if self.fatal:
            yield StreamEvent(finished=True, finish_reason="error", error=self.fatal)
            return
        rid = request_id or "req-" + uuid.uuid4().hex[:16]
        live = _Live(asyncio.get_running_loop(), IncrementalDetokenizer(self.tokenizer), list(params.stop))
        self._live[rid] = live
        self._in.put(("add", rid, list(prompt_ids), params))
        try:
            while True:
                ev: StreamEvent = await live.q.get()
                yield ev
                if ev.finished:
                    break
        finally:
            if rid in self._live:               # client went away
                self._in.put(("abort", rid, None, None))
                self._live.pop(rid, None)

    # ---- scheduler thread
    def _emit(self, rid: str, ev: StreamEvent) -> None:
        live = self._live.get(rid)
        if live is not None:
            live.loop.call_soon_threadsafe(live.q.put_nowait, ev)

    def _handle_output(self, o) -> None:
        live = self._live.get(o.request_id)
        if live is None:
            return
        if live.t_first is None and o.new_token_ids:
            live.t_first = time.time()
        text = live.detok.push(o.new_token_ids) if o.new_token_ids else ""
        finished, reason = o.finished, o.finish_reason
        if live.stops:
            buf = live.held + text
            cut = min((i for i in (buf.find(s) for s in live.stops) if i >= 0), default=-1)
            if cut >= 0:
                text, live.held = buf[:cut], ""
                finished, reason = True, "stop"
                self.engine.abort(o.request_id)
            else:
                keep = 0
                for s in live.stops:
                    for k in range(min(len(s) - 1, len(buf)), 0, -1):
                        if s.startswith(buf[-k:]):
                            keep = max(keep, k)
                            break
                text, live.held = (buf[:len(buf) - keep], buf[len(buf) - keep:]) if keep else (buf, "")
        if finished:
            text += live.detok.flush() + ("" if reason == "stop" else live.held)
        usage = None
        if finished:
            now = time.time()
            ttft = (live.t_first - live.t0) * 1e3 if live.t_first else None
            dec = (now - live.t_first) * 1e3 if live.t_first else None
            n = len(o.output_ids)
            usage = {"prompt_tokens": o.prompt_tokens, "completion_tokens": n, "total_tokens": o.prompt_tokens + n,
                     "prompt_tokens_details": {"cached_tokens": o.cached_tokens},
                     "completion_tokens_details": {"reasoning_tokens": 0,
                                                   "accepted_prediction_tokens": o.accepted_draft_tokens,
                                                   "rejected_prediction_tokens": o.rejected_draft_tokens},
                     "time_to_first_token_ms": ttft, "decode_time_ms": dec,
                     "total_time_ms": (now - live.t0) * 1e3,
                     "response_tokens_per_second": (n / (dec / 1e3)) if dec and dec > 0 else None}
        self._emit(o.request_id, StreamEvent(text, list(o.new_token_ids), finished, reason, usage, o.logprobs))
        if finished:
            self._live.pop(o.request_id, None)

    def request_swap(self, build, timeout_s: float = 600.0):
        """Replace the engine without closing the listener: `build()` returns the new engine (and
        optionally a tokenizer) and runs on the scheduler thread once nothing is in flight, so no
        step ever sees two models. New requests queue behind the swap. Returns the new engine or
        raises what `build` raised (the old engine then keeps serving). Role of the reference's
        model hot-swap (``crates/server/src/main_modules/model_swap.rs``)."""
        done = threading.Event()
        box = {}
        self._in.put(("swap", None, (build, box, done), None))
        if not done.wait(timeout_s):
            raise TimeoutError("model swap did not finish in time")
        if "error" in box:
            raise box["error"]
        return box["engine"]

    def _swap(self, payload) -> None:
        build, box, done = payload
        try:
            old = self.engine.target() if hasattr(self.engine, "target") else self.engine
            old.flush() if hasattr(old, "flush") else None
            res = build()
            new, tok = res if isinstance(res, tuple) else (res, None)
            if hasattr(self.engine, "swap"):
                self.engine.swap(new)
            else:
                self.engine = new
            if tok is not None:
                if hasattr(self.tokenizer, "swap"):
                    self.tokenizer.swap(tok)
                else:
                    self.tokenizer = tok
            box["engine"] = new
            del old
            import gc
            gc.collect()
            try:
                import torch
                if torch.cuda.is_available():
                    torch.cuda.empty_cache()
            except Exception:
                pass
        except Exception as e:
            box["error"] = e
        finally:
            done.set()

    def _run(self) -> None:
        eng = self.engine
        pending_swap = None
        while not self._stop.is_set():
            try:
                if pending_swap is not None and not eng.has_work():
                    self._swap(pending_swap)
                    pending_swap = None
                    eng = self.engine
                block = not eng.has_work()
                ops = []
                while True:
                    try:
                        ops.append(self._in.get(timeout=0.05) if block else self._in.get_nowait())
                    except queue.Empty:
                        break
                    block = False
                if self.control is not None:
                    self.control.check_peers()
                    ops = self.control.exchange(ops)
                if pending_swap is not None:
                    # requests that arrive while the old engine drains wait for the new one
                    held = [o for o in ops if o[0] == "add"]
                    ops = [o for o in ops if o[0] != "add"]
                    for o in held:
                        self._in.put(o)
                    if held and not eng.has_work():
                        continue
                for kind, rid, ids, params in ops:
                    if kind == "swap":
                        pending_swap = ids
                        continue
                    if kind == "add":
                        try:
                            eng.add_request(ids, params, request_id=rid, **({"images": params.images} if getattr(params, "images", None) else {}))
                        except Exception as e:          # bad request: answer it, keep serving
                            self._emit(rid, StreamEvent(finished=True, finish_reason="error", error=str(e)))
                            self._live.pop(rid, None)
                    elif kind == "abort":
                        eng.abort(rid)
                if eng.has_work():
                    for o in eng.step():
                        self._handle_output(o)
            except Exception as e:                      # device fault: latch, fail everything
                self.fatal = f"{type(e).__name__}: {e}"
                for rid in list(self._live):
                    self._emit(rid, StreamEvent(finished=True, finish_reason="error", error=self.fatal))
                self._live.clear()
                return
