"""Token-bucket rate limiter keyed by API key / client address
(role of ``crates/server/src/rate_limiter*``)."""
from __future__ import annotations

import time
from typing import Dict, Tuple


class RateLimiter:
    def __init__(self, rate_per_s: float = 0.0, burst: int = 0, clock=time.monotonic):
        self.rate, self.burst, self.clock = rate_per_s, burst or max(1, int(rate_per_s)), clock
        self._b: Dict[str, Tuple[float, float]] = {}

    def allow(self, key: str) -> bool:
        if self.rate <= 0:
            return True
        now = self.clock()
        tokens, last = self._b.get(key, (float(self.burst), now))
        tokens = min(self.burst, tokens + (now - last) * self.rate)
        if tokens < 1.0:
            self._b[key] = (tokens, now)
            return False
        self._b[key] = (tokens - 1.0, now)
        return True
