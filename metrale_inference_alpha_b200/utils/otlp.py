"""OTLP/HTTP JSON export of the telemetry hub (``POST <endpoint>/v1/metrics``): counters become
cumulative monotonic sums, gauges gauges, the millisecond histograms explicit-bucket histograms.
``OtlpExporter`` pushes on a period from a daemon thread; a failed push is counted and dropped
(the serving loop never waits on the collector). Only the standard library is used.

Role of the reference's ``crates/telemetry/src/export/otlp.rs``.
"""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from typing import Dict, Optional

from .telemetry import _BUCKETS, Telemetry

_UNITS = {"tokens": "{token}", "requests": "{request}", "steps": "{step}", "replays": "{replay}", "bytes": "By",
          "blocks": "{block}", "ms": "ms", "joules": "J", "watts": "W"}


def _unit(name: str) -> str:
    for k, u in _UNITS.items():
        if k in name:
            return u
    return "1"


def metrics_body(tel: Telemetry, extra_gauges: Optional[Dict[str, float]] = None, service: str = "metrale-b200",
                 now_ns: Optional[int] = None) -> dict:
    """The ExportMetricsServiceRequest of the hub's current state, as a JSON-able dict."""
    now = str(now_ns if now_ns is not None else time.time_ns())
    start = str(int(tel.start * 1e9))
    metrics = []
    with tel._lock:
        counters = dict(tel.counters)
        hist = {k: list(v) for k, v in tel.hist.items()}
        hsum = dict(tel.hist_sum)
    for k, v in sorted(counters.items()):
        point = {"startTimeUnixNano": start, "timeUnixNano": now}
        if float(v).is_integer():
            point["asInt"] = str(int(v))
        else:
            point["asDouble"] = float(v)
        metrics.append({"name": f"metrale.{k}", "unit": _unit(k),
                        "sum": {"aggregationTemporality": 2, "isMonotonic": True, "dataPoints": [point]}})
    for k, v in sorted({**tel.gauges, **(extra_gauges or {})}.items()):
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            metrics.append({"name": f"metrale.{k}", "unit": _unit(k),
                            "gauge": {"dataPoints": [{"timeUnixNano": now, "asDouble": float(v)}]}})
    for k, h in sorted(hist.items()):
        metrics.append({"name": f"metrale.{k}", "unit": "ms", "histogram": {
            "aggregationTemporality": 2,
            "dataPoints": [{"startTimeUnixNano": start, "timeUnixNano": now, "count": str(sum(h)),
                            "sum": float(hsum.get(k, 0.0)), "bucketCounts": [str(n) for n in h],
                            "explicitBounds": [float(b) for b in _BUCKETS]}]}})
    return {"resourceMetrics": [{
        "resource": {"attributes": [{"key": "service.name", "value": {"stringValue": service}}]},
        "scopeMetrics": [{"scope": {"name": "metrale_inference_alpha_b200.telemetry"}, "metrics": metrics}]}]}


def push(endpoint: str, body: dict, timeout: float = 2.0, headers: Optional[Dict[str, str]] = None) -> int:
    url = endpoint.rstrip("/")
    if not url.endswith("/v1/metrics"):
        url += "/v1/metrics"
    req = urllib.request.Request(url, data=json.dumps(body).encode(), method="POST",
                                 headers={"Content-Type": "application/json", **(headers or {})})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return r.status


class OtlpExporter:
    def __init__(self, tel: Telemetry, endpoint: str, period_s: float = 10.0, gauges=None, service: str = "metrale-b200",
                 headers: Optional[Dict[str, str]] = None):
        self.tel, self.endpoint, self.period, self.gauges = tel, endpoint, period_s, gauges
        self.service, self.headers = service, headers
        self.pushed = self.failed = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def export_once(self) -> bool:
        try:
            extra = self.gauges() if callable(self.gauges) else self.gauges
            push(self.endpoint, metrics_body(self.tel, extra, self.service), headers=self.headers)
            self.pushed += 1
            return True
        except Exception:
            self.failed += 1
            return False

    def start(self) -> "OtlpExporter":
        def loop():
            while not self._stop.wait(self.period):
                self.export_once()
        self._thread = threading.Thread(target=loop, name="otlp-export", daemon=True)
        self._thread.start()
        return self

    def stop(self, final_push: bool = True) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        if final_push:
            self.export_once()
