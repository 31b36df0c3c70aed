"""MTP throughput arbiter: measures tokens/s with speculation on and off in windows of steps
and keeps the faster mode, with a margin and a dwell so it does not flap.
(``crates/speculative/src/mtp_gate.rs``: windows of 16 steps, EWMA tok/s per mode, 5 % margin,
2-window dwell.)"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SpecStats:
    steps: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0

    @property
    def accept_len(self) -> float:
        return self.emitted / self.steps if self.steps else 0.0

    @property
    def accept_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0


class MtpGate:
    MEASURE_DECODE, MEASURE_VERIFY = "decode", "verify"

    def __init__(self, window: int = 16, margin: float = 0.05, dwell: int = 2, alpha: float = 0.5,
                 reprobe_windows: int = 32, enabled: bool = True):
        self.window, self.margin, self.dwell, self.alpha = window, margin, dwell, alpha
        self.reprobe_windows = reprobe_windows
        self.enabled = enabled
        self.mode = self.MEASURE_VERIFY if enabled else self.MEASURE_DECODE
        self.ewma = {self.MEASURE_DECODE: None, self.MEASURE_VERIFY: None}
        self._tokens = 0
        self._time = 0.0
        self._steps = 0
        self._windows_in_mode = 0
        self._since_probe = 0
        self.switches = 0

    def next_step(self) -> str:
        """Mode for the next decode-lane step."""
        return self.mode if self.enabled else self.MEASURE_DECODE

    def record(self, tokens: int, seconds: float) -> None:
        if not self.enabled:
            return
        self._tokens += tokens
        self._time += seconds
        self._steps += 1
        if self._steps < self.window:
            return
        rate = self._tokens / self._time if self._time > 0 else 0.0
        prev = self.ewma[self.mode]
        self.ewma[self.mode] = rate if prev is None else self.alpha * rate + (1 - self.alpha) * prev
        self._tokens, self._time, self._steps = 0, 0.0, 0
        self._windows_in_mode += 1
        self._since_probe += 1
        other = self.MEASURE_DECODE if self.mode == self.MEASURE_VERIFY else self.MEASURE_VERIFY
        if self.ewma[other] is None:
            if self._windows_in_mode >= self.dwell:
                self._switch(other)                         # first measurement of the other mode
            return
        if self._windows_in_mode < self.dwell:
            return
        if self.ewma[other] > self.ewma[self.mode] * (1 + self.margin):
            self._switch(other)
        elif self._since_probe >= self.reprobe_windows:
            self.ewma[other] = None                         # stale: measure it again next dwell
            self._since_probe = 0

    def _switch(self, mode: str) -> None:
        self.mode = mode
        self._windows_in_mode = 0
        self.switches += 1
