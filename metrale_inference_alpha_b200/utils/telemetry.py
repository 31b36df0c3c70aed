"""Level-gated telemetry hub: counters, histograms and lane spans, exported as Prometheus text.
At level "off" every hook is one attribute test. Level "kernel" additionally times scheduler
lanes with CUDA events. Role of ``crates/telemetry`` (``level.rs``, ``hub.rs``,
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
        assert level in LEVELS
        self.level = level
        self.enabled = level != "off"
        self._lock = threading.Lock()
        self.counters: Dict[str, float] = defaultdict(float)
        self.gauges: Dict[str, float] = {}
        self.hist: Dict[str, List[int]] = {}
        self.hist_sum: Dict[str, float] = defaultdict(float)
        self.start = time.time()

    def inc(self, name: str, v: float = 1.0) -> None:
        if self.enabled:
            with self._lock:
                self.counters[name] += v

    def set(self, name: str, v: float) -> None:
        if self.enabled:
            self.gauges[name] = v

    def observe_ms(self, name: str, ms: float) -> None:
        if not self.enabled:
            return
        with self._lock:
            h = self.hist.setdefault(name, [0] * (len(_BUCKETS) + 1))
            h[bisect.bisect_left(_BUCKETS, ms)] += 1
            self.hist_sum[name] += ms

    def span(self, name: str):
        return _Span(self, name)

    def prometheus(self, extra: Dict[str, float] = None) -> str:
        lines = [f"# metrale b200 engine, telemetry level {self.level}",
                 f"metrale_uptime_seconds {time.time() - self.start:.1f}"]
        for k, v in sorted(self.counters.items()):
            lines.append(f"metrale_{k}_total {v:g}")
        for k, v in sorted({**self.gauges, **(extra or {})}.items()):
            if isinstance(v, (int, float)):
                lines.append(f"metrale_{k} {v:g}")
        for k, h in sorted(self.hist.items()):
            acc = 0
            for b, n in zip(_BUCKETS, h):
                acc += n
                lines.append(f'metrale_{k}_ms_bucket{{le="{b}"}} {acc}')
            lines.append(f'metrale_{k}_ms_bucket{{le="+Inf"}} {acc + h[-1]}')
            lines.append(f"metrale_{k}_ms_sum {self.hist_sum[k]:g}")
            lines.append(f"metrale_{k}_ms_count {acc + h[-1]}")
        return "\n".join(lines) + "\n"


class _Span:
    def __init__(self, t: Telemetry, name: str):
        self.t, self.name = t, name

    def __enter__(self):
        self.t0 = time.perf_counter() if self.t.enabled else 0.0
        return self

    def __exit__(self, *exc):
        if self.t.enabled:
            self.t.observe_ms(self.name, (time.perf_counter() - self.t0) * 1e3)
        return False
