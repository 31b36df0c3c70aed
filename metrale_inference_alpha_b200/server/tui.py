"""Terminal front end for a running server: a live dashboard (model, throughput, queue, KV pool,
latency percentiles, devices) and a streaming chat with slash commands.

    metrale-b200 tui  --url http://127.0.0.1:8888        # dashboard, refreshes every second
    metrale-b200 chat --url http://127.0.0.1:8888        # chat; /help lists the commands

Both talk to the public HTTP surface only (``/metrics``, ``/health``, ``/forward``, ``/hardware``,
``/v1/chat/completions``), through a small transport object so that tests can drive them against
an in-process app. Rendering uses ``rich``.

Role of the reference's ``crates/server/src/tui`` (dashboard, chat, chat_stream, chat_thinking).
"""
from __future__ import annotations

import json
import re
import time
import urllib.request
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Tuple

_LINE = re.compile(r'^([a-zA-Z_:][a-zA-Z0-9_:]*)(\{[^}]*\})?\s+([-+0-9.eEinfa]+)\s*$')


def parse_prometheus(text: str) -> Dict[str, float]:
    """Prometheus text -> {name or name{labels}: value}; comments and malformed lines are skipped."""
    out: Dict[str, float] = {}
    for ln in text.splitlines():
        m = _LINE.match(ln.strip())
        if m:
            try:
                out[m.group(1) + (m.group(2) or "")] = float(m.group(3))
            except ValueError:
                pass
    return out


def histogram_quantile(metrics: Dict[str, float], name: str, q: float) -> Optional[float]:
    """Quantile of a ``<name>_bucket{le=...}`` histogram by linear interpolation inside the bucket."""
    pts: List[Tuple[float, float]] = []
    for k, v in metrics.items():
        if k.startswith(name + "_bucket{"):
            le = k.split('le="', 1)[1].split('"', 1)[0]
            pts.append((float("inf") if le == "+Inf" else float(le), v))
    pts.sort()
    if not pts or pts[-1][1] <= 0:
        return None
    want = q * pts[-1][1]
    lo_b, lo_c = 0.0, 0.0
    for b, c in pts:
        if c >= want:
            if b == float("inf"):
                return lo_b
            return lo_b + (b - lo_b) * ((want - lo_c) / max(c - lo_c, 1e-9))
        lo_b, lo_c = b, c
    return pts[-1][0]


class HttpTransport:
    def __init__(self, base: str, api_key: Optional[str] = None, timeout: float = 5.0):
        self.base, self.key, self.timeout = base.rstrip("/"), api_key, timeout

    def _req(self, path: str, body: Optional[dict] = None):
        headers = {"Content-Type": "application/json"}
        if self.key:
            headers["Authorization"] = f"Bearer {self.key}"
        data = json.dumps(body).encode() if body is not None else None
        return urllib.request.urlopen(urllib.request.Request(self.base + path, data=data, headers=headers),
                                      timeout=self.timeout if body is None else 600)

    def get_text(self, path: str) -> str:
        with self._req(path) as r:
            return r.read().decode("utf-8", "replace")

    def post_stream(self, path: str, body: dict) -> Iterator[str]:
        with self._req(path, body) as r:
            for raw in r:
                yield raw.decode("utf-8", "replace").rstrip("\n")


# ----------------------------------------------------------------------------- dashboard
@dataclass
class Sample:
    at: float
    metrics: Dict[str, float]


class Dashboard:
    """Polls the server and turns consecutive samples into rates."""

    def __init__(self, transport, clock: Callable[[], float] = time.time):
        self.t, self.clock = transport, clock
        self.prev: Optional[Sample] = None
        self.cur: Optional[Sample] = None
        self.forward: Dict[str, object] = {}
        self.hardware: Dict[str, object] = {}
        self.error: Optional[str] = None
        self.history: List[float] = []                   # tok/s of the last minute

    def _json(self, path: str) -> dict:
        try:
            return json.loads(self.t.get_text(path))
        except Exception:
            return {}

    def poll(self) -> None:
        try:
            m = parse_prometheus(self.t.get_text("/metrics"))
            self.error = None
        except Exception as e:
            self.error = f"{type(e).__name__}: {e}"
            return
        self.prev, self.cur = self.cur, Sample(self.clock(), m)
        if not self.forward:
            self.forward = self._json("/forward")
        if not self.hardware:
            self.hardware = self._json("/hardware")
        r = self.rate("metrale_decode_tokens_total")
        if r is not None:
            self.history = (self.history + [r])[-60:]

    def value(self, name: str, default: float = 0.0) -> float:
        return self.cur.metrics.get(name, default) if self.cur else default

    def rate(self, name: str) -> Optional[float]:
        if not self.prev or not self.cur or name not in self.cur.metrics:
            return None
        dt = self.cur.at - self.prev.at
        # a counter that did not exist at the previous sample started from zero since then
        return max(0.0, (self.cur.metrics[name] - self.prev.metrics.get(name, 0.0)) / dt) if dt > 0 else None

    def summary(self) -> Dict[str, object]:
        m = self.cur.metrics if self.cur else {}
        q = lambda name, p: histogram_quantile(m, name, p)
        return {
            "model": self.forward.get("model"), "arch": self.forward.get("arch"),
            "weights": self.forward.get("weight_format"), "kv": self.forward.get("kv_dtype"),
            "decode_tok_s": self.rate("metrale_decode_tokens_total"),
            "prefill_tok_s": self.rate("metrale_prefill_tokens_total"),
            "req_s": self.rate("metrale_http_requests_total"),
            "running": self.value("metrale_engine_running"), "waiting": self.value("metrale_engine_waiting"),
            "free_blocks": self.value("metrale_engine_free_blocks"), "preempted": self.value("metrale_engine_preempted"),
            "ttft_p50_ms": q("metrale_ttft_ms", 0.5), "ttft_p99_ms": q("metrale_ttft_ms", 0.99),
            "http_p50_ms": q("metrale_http_latency_ms", 0.5), "http_p99_ms": q("metrale_http_latency_ms", 0.99),
            "uptime_s": self.value("metrale_uptime_seconds"), "error": self.error,
        }

    def render(self):
        from rich.console import Group
        from rich.panel import Panel
        from rich.table import Table
        s = self.summary()
        f = lambda v, unit="", nd=1: "-" if v is None else f"{v:,.{nd}f}{unit}"
        head = Table.grid(padding=(0, 2))
        head.add_row("model", str(s["model"] or "?"), "arch", str(s["arch"] or "?"), "weights", str(s["weights"] or "?"),
                     "kv", str(s["kv"] or "?"), "up", f(s["uptime_s"], " s", 0))
        load = Table(title="load", expand=True)
        for c in ("decode tok/s", "prefill tok/s", "req/s", "running", "waiting", "free KV blocks", "preempted"):
            load.add_column(c, justify="right")
        load.add_row(f(s["decode_tok_s"]), f(s["prefill_tok_s"]), f(s["req_s"], nd=2), f(s["running"], nd=0),
                     f(s["waiting"], nd=0), f(s["free_blocks"], nd=0), f(s["preempted"], nd=0))
        lat = Table(title="latency", expand=True)
        for c in ("TTFT p50", "TTFT p99", "HTTP p50", "HTTP p99"):
            lat.add_column(c, justify="right")
        lat.add_row(f(s["ttft_p50_ms"], " ms"), f(s["ttft_p99_ms"], " ms"), f(s["http_p50_ms"], " ms"), f(s["http_p99_ms"], " ms"))
        parts = [Panel(head, title="metrale b200"), load, lat, Panel(sparkline(self.history), title="decode tok/s, last minute")]
        devs = self.hardware.get("devices") or []
        if devs:
            dt = Table(title="devices", expand=True)
            for c in ("#", "name", "SMs", "total GB", "free GB"):
                dt.add_column(c)
            for d in devs:
                dt.add_row(str(d.get("index")), str(d.get("name")), str(d.get("sms")), str(d.get("total_gb")), str(d.get("free_gb")))
            parts.append(dt)
        if s["error"]:
            parts.append(Panel(f"[red]{s['error']}[/red]", title="server unreachable"))
        return Group(*parts)

    def run(self, period_s: float = 1.0, iterations: Optional[int] = None) -> None:
        from rich.live import Live
        n = 0
        with Live(self.render(), refresh_per_second=4, screen=False) as live:
            while iterations is None or n < iterations:
                self.poll()
                live.update(self.render())
                n += 1
                time.sleep(period_s)


def sparkline(values: List[float], width: int = 60) -> str:
    if not values:
        return "(no samples yet)"
    bars = "▁▂▃▄▅▆▇█"
    vals = values[-width:]
    hi = max(vals) or 1.0
    return "".join(bars[min(7, int(7 * v / hi))] for v in vals) + f"  peak {hi:,.0f}"


# ----------------------------------------------------------------------------- chat
HELP = """/help                this text
/clear               forget the conversation
/system <text>       set (or with no text: remove) the system prompt
/thinking on|off     ask the model to reason before answering
/temp <t>            sampling temperature          /max <n>   max tokens per answer
/stats               tokens and speed of the last answer
/save <file>         write the conversation as JSON
/quit                leave"""


@dataclass
class ChatSession:
    """Conversation state + one streaming request per user turn. `emit(kind, text)` receives the
    pieces as they arrive: kind is "reasoning", "content", "tool" or "info"."""
    transport: object
    model: str = "default"
    system: Optional[str] = None
    thinking: bool = False
    temperature: float = 0.7
    max_tokens: int = 1024
    messages: List[dict] = field(default_factory=list)
    last_usage: Optional[dict] = None
    last_seconds: float = 0.0

    def command(self, line: str, emit: Callable[[str, str], None]) -> bool:
        """Handles a slash command; returns False when the session should end."""
        cmd, _, arg = line.strip().partition(" ")
        arg = arg.strip()
        if cmd in ("/quit", "/exit", "/q"):
            return False
        if cmd == "/help":
            emit("info", HELP)
        elif cmd == "/clear":
            self.messages.clear()
            emit("info", "conversation cleared")
        elif cmd == "/system":
            self.system = arg or None
            emit("info", "system prompt " + ("set" if arg else "removed"))
        elif cmd == "/thinking":
            self.thinking = arg.lower() in ("on", "1", "true", "yes")
            emit("info", f"thinking {'on' if self.thinking else 'off'}")
        elif cmd == "/temp":
            try:
                self.temperature = max(0.0, float(arg))
                emit("info", f"temperature {self.temperature}")
            except ValueError:
                emit("info", "usage: /temp <number>")
        elif cmd == "/max":
            try:
                self.max_tokens = max(1, int(arg))
                emit("info", f"max tokens {self.max_tokens}")
            except ValueError:
                emit("info", "usage: /max <integer>")
        elif cmd == "/stats":
            u = self.last_usage or {}
            n = u.get("completion_tokens")
            if n:
                emit("info", f"{u.get('prompt_tokens')} prompt + {n} completion tokens in {self.last_seconds:.2f} s "
                             f"({n / max(self.last_seconds, 1e-9):.1f} tok/s), TTFT {u.get('time_to_first_token_ms', '?')} ms")
            else:
                emit("info", "no answer yet")
        elif cmd == "/save":
            if not arg:
                emit("info", "usage: /save <file>")
            else:
                with open(arg, "w") as f:
                    json.dump({"system": self.system, "messages": self.messages}, f, indent=1)
                emit("info", f"saved {len(self.messages)} messages to {arg}")
        else:
            emit("info", f"unknown command {cmd}; /help lists them")
        return True

    def ask(self, text: str, emit: Callable[[str, str], None]) -> str:
        self.messages.append({"role": "user", "content": text})
        msgs = ([{"role": "system", "content": self.system}] if self.system else []) + self.messages
        body = {"model": self.model, "messages": msgs, "stream": True, "stream_options": {"include_usage": True},
                "temperature": self.temperature, "max_tokens": self.max_tokens, "enable_thinking": self.thinking}
        t0 = time.time()
        content, calls = [], {}
        try:
            for line in self.transport.post_stream("/v1/chat/completions", body):
                if not line.startswith("data: "):
                    continue
                data = line[6:]
                if data == "[DONE]":
                    break
                d = json.loads(data)
                if "error" in d:
                    emit("info", f"error: {d['error'].get('message')}")
                    break
                if d.get("usage"):
                    self.last_usage = d["usage"]
                for ch in d.get("choices") or []:
                    delta = ch.get("delta") or {}
                    if delta.get("reasoning_content"):
                        emit("reasoning", delta["reasoning_content"])
                    if delta.get("content"):
                        content.append(delta["content"])
                        emit("content", delta["content"])
                    for tc in delta.get("tool_calls") or []:
                        slot = calls.setdefault(tc.get("index", 0), {"name": "", "arguments": ""})
                        fn = tc.get("function") or {}
                        slot["name"] += fn.get("name") or ""
                        slot["arguments"] += fn.get("arguments") or ""
        except Exception as e:
            emit("info", f"request failed: {type(e).__name__}: {e}")
            self.messages.pop()
            return ""
        self.last_seconds = time.time() - t0
        for c in calls.values():
            emit("tool", f"{c['name']}({c['arguments']})")
        answer = "".join(content)
        self.messages.append({"role": "assistant", "content": answer})
        return answer

    def repl(self, read: Callable[[str], str] = input, console=None) -> None:
        from rich.console import Console
        con = console or Console()
        styles = {"reasoning": "dim italic", "content": "", "tool": "yellow", "info": "cyan"}

        def emit(kind, text):
            con.print(text, style=styles.get(kind, ""), end="" if kind in ("reasoning", "content") else "\n",
                      markup=False, highlight=False)
        con.print("metrale b200 chat: /help for commands", style="cyan")
        while True:
            try:
                line = read("\n> ")
            except (EOFError, KeyboardInterrupt):
                break
            if not line.strip():
                continue
            if line.startswith("/"):
                if not self.command(line, emit):
                    break
                continue
            self.ask(line, emit)
            con.print()
