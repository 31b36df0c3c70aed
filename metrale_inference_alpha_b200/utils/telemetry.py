"""Level-gated telemetry hub: counters, histograms and lane spans, exported as Prometheus text.
At level "off" every hook is one attribute test. At level "basic" spans are host timers. At
level "kernel" (on a CUDA device) spans are pairs of CUDA events recorded on the launching
stream and resolved later without synchronising, and every kernel launcher of ``ops`` leaves
an event behind it, so consecutive events give per-kernel device time (``kernel_<name>_us``
histograms; launches inside a replayed CUDA graph are one span, the graph's). Role of
``crates/telemetry`` (``level.rs``, ``hub.rs``, ``kernel.rs:3-15`` per-kernel spans,
``export/prometheus*.rs``) and ``server/src/metrics.rs``."""
from __future__ import annotations

import bisect
import threading
import time
from collections import defaultdict
from typing import Dict, List

LEVELS = ("off", "basic", "kernel")
_BUCKETS = [1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 30000]


class Telemetry:
    def __init__(self, level: str = "off"):
        level = "kernel" if level == "full" else level
        assert level in LEVELS
        self.level = level
        self.enabled = level != "off"
        self._lock = threading.Lock()
        self.counters: Dict[str, float] = defaultdict(float)
        self.gauges: Dict[str, float] = {}
        self.hist: Dict[str, List[int]] = {}
        self.hist_sum: Dict[str, float] = defaultdict(float)
        self.start = time.time()
        self._pending = []               # (name, start event, end event) not yet resolved
        self._launches = []              # (kernel name, event recorded after its launch)
        self._cuda = False
        if level == "kernel":
            try:
                import torch
                self._cuda = torch.cuda.is_available()
            except Exception:
                self._cuda = False
            if self._cuda:
                from ..ops import _native
                _native.set_launch_hook(self._on_launch)

    def close(self) -> None:
        """Detach the per-kernel hook (tests; a second hub in the same process)."""
        if self._cuda:
            from ..ops import _native
            _native.set_launch_hook(None)
            self._cuda = False

    # ------------------------------------------------------------------ CUDA-event timing
    def _on_launch(self, name: str) -> None:
        import torch
        if torch.cuda.is_current_stream_capturing():
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._launches.append((name, ev))
        if len(self._launches) > 2048:
            self.resolve()

    def resolve(self) -> None:
        """Turn finished event pairs into observations; never blocks."""
        keep = []
        for name, a, b in self._pending:
            if b.query():
                self.observe_ms(name, a.elapsed_time(b))
            else:
                keep.append((name, a, b))
        self._pending = keep
        ls = self._launches
        i = 1
        while i < len(ls) and ls[i][1].query():
            self.observe_ms(f"kernel_{ls[i][0]}", ls[i - 1][1].elapsed_time(ls[i][1]), unit_us=True)
            i += 1
        if i > 1:
            self._launches = ls[i - 1:]

    def inc(self, name: str, v: float = 1.0) -> None:
        if self.enabled:
            with self._lock:
                self.counters[name] += v

    def set(self, name: str, v: float) -> None:
        if self.enabled:
            self.gauges[name] = v

    def observe_ms(self, name: str, ms: float, unit_us: bool = False) -> None:
        """One observation in milliseconds (`unit_us`: stored and bucketed in microseconds under <name>_us)."""
        if not self.enabled:
            return
        if unit_us:
            name, ms = name + "_us", ms * 1e3
        with self._lock:
            h = self.hist.setdefault(name, [0] * (len(_BUCKETS) + 1))
            h[bisect.bisect_left(_BUCKETS, ms)] += 1
            self.hist_sum[name] += ms

    def span(self, name: str):
        return _Span(self, name)

    def prometheus(self, extra: Dict[str, float] = None) -> str:
        if self._cuda:
            self.resolve()
        lines = [f"# metrale b200 engine, telemetry level {self.level}",
                 f"metrale_uptime_seconds {time.time() - self.start:.1f}"]
        for k, v in sorted(self.counters.items()):
            lines.append(f"metrale_{k}_total {v:g}")
        for k, v in sorted({**self.gauges, **(extra or {})}.items()):
            if isinstance(v, (int, float)):
                lines.append(f"metrale_{k} {v:g}")
        for k, h in sorted(self.hist.items()):
            acc = 0
            name = k if k.endswith("_us") else k + "_ms"     # microsecond series carry their own unit suffix
            for b, cnt in zip(_BUCKETS, h):
                acc += cnt
                lines.append(f'metrale_{name}_bucket{{le="{b}"}} {acc}')
            lines.append(f'metrale_{name}_bucket{{le="+Inf"}} {acc + h[-1]}')
            lines.append(f"metrale_{name}_sum {self.hist_sum[k]:g}")
            lines.append(f"metrale_{name}_count {acc + h[-1]}")
        return "\n".join(lines) + "\n"


class _Span:
    def __init__(self, t: Telemetry, name: str):
        self.t, self.name = t, name

    def __enter__(self):
        t = self.t
        self.ev = None
        if t._cuda:
            import torch
            if not torch.cuda.is_current_stream_capturing():
                self.ev = torch.cuda.Event(enable_timing=True)
                self.ev.record()
        self.t0 = time.perf_counter() if t.enabled else 0.0
        return self

    def __exit__(self, *exc):
        t = self.t
        if self.ev is not None:
            import torch
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            t._pending.append((self.name, self.ev, end))      # device time of the lane, resolved later
            if len(t._pending) > 256:
                t.resolve()
        elif t.enabled:
            t.observe_ms(self.name, (time.perf_counter() - self.t0) * 1e3)
        return False
