"""Process-wide GPU fault latch: the first reason wins; once set, the engine refuses new work,
``/health`` fails and the server exits with code 70 after draining.
Role of ``crates/core/src/fault.rs:36-105`` and ``gpu-runtime/src/cuda_backend/fault_probe.rs``."""
from __future__ import annotations

import threading
from typing import Optional

EXIT_CODE_GPU_FAULT = 70


class FaultLatch:
    def __init__(self):
        self._lock = threading.Lock()
        self._reason: Optional[str] = None

    def set(self, reason: str) -> bool:
        with self._lock:
            if self._reason is None:
                self._reason = reason
                return True
            return False

    def is_set(self) -> bool:
        return self._reason is not None

    def reason(self) -> Optional[str]:
        return self._reason


def probe_device(device) -> Optional[str]:
    """After a failed launch: is the context still usable? Returns the error text when a
    stream synchronize fails (context lost), else None."""
    import torch
    try:
        torch.cuda.synchronize(device)
        return None
    except RuntimeError as e:      # pragma: no cover - needs a faulted GPU
        return str(e)
