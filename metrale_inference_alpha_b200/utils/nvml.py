"""Device sampler over NVML: SM / memory clocks, power, temperature, utilisation, memory in use and
the throttle reasons, sampled on a background thread; integrates power into energy so that a span
(a request, a benchmark rung) can be charged joules per token. Read-only: nothing here changes a
clock, a power limit or any other device setting. The NVML binding is injectable so that tests run
against a fake. Role of the reference's NVML device sampler + energy attribution
(``crates/telemetry/src/device.rs``, ``crates/gpu-sys/src/nvml.rs``)."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
           0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
           0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
BAD_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")


@dataclass
class DeviceSample:
    t: float
    sm_mhz: int
    mem_mhz: int
    power_w: float
    temp_c: int
    util_pct: int
    mem_used_bytes: int
    reasons: List[str] = field(default_factory=list)


def decode_reasons(mask: int) -> List[str]:
    return [name for bit, name in REASONS.items() if mask & bit and name != "gpu_idle"]


class DeviceSampler:
    def __init__(self, index: int = 0, period_s: float = 0.2, nvml=None, clock=time.monotonic):
        if nvml is None:
            import pynvml as nvml                      # provided by nvidia-ml-py
        self.nvml, self.index, self.period, self.clock = nvml, index, period_s, clock
        self.samples: List[DeviceSample] = []
        self.energy_j = 0.0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._h = None

    def _handle(self):
        if self._h is None:
            self.nvml.nvmlInit()
            self._h = self.nvml.nvmlDeviceGetHandleByIndex(self.index)
        return self._h

    def sample_once(self) -> DeviceSample:
        n, h = self.nvml, self._handle()
        s = DeviceSample(
            t=self.clock(),
            sm_mhz=int(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)),
            mem_mhz=int(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_MEM)),
            power_w=n.nvmlDeviceGetPowerUsage(h) / 1000.0,
            temp_c=int(n.nvmlDeviceGetTemperature(h, n.NVML_TEMPERATURE_GPU)),
            util_pct=int(n.nvmlDeviceGetUtilizationRates(h).gpu),
            mem_used_bytes=int(n.nvmlDeviceGetMemoryInfo(h).used),
            reasons=decode_reasons(int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
        if self.samples:
            prev = self.samples[-1]
            self.energy_j += 0.5 * (prev.power_w + s.power_w) * max(0.0, s.t - prev.t)   # trapezoid
        self.samples.append(s)
        return s

    def start(self) -> None:
        def run():
            while not self._stop.is_set():
                try:
                    self.sample_once()
                except Exception:
                    return
                self._stop.wait(self.period)
        self._thread = threading.Thread(target=run, name="nvml-sampler", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, tokens: int = 0) -> Dict[str, object]:
        if not self.samples:
            return {"samples": 0}
        sm = sorted(s.sm_mhz for s in self.samples)
        reasons = sorted({r for s in self.samples for r in s.reasons})
        out = {"samples": len(self.samples), "sm_mhz_median": sm[len(sm) // 2], "sm_mhz_min": sm[0],
               "power_w_max": max(s.power_w for s in self.samples), "temp_c_max": max(s.temp_c for s in self.samples),
               "energy_j": round(self.energy_j, 3), "reasons": reasons,
               "rejected": any(r in BAD_REASONS for r in reasons)}
        if tokens > 0:
            out["joules_per_token"] = self.energy_j / tokens
        return out
