"""NVTX ranges around engine phases (scheduler step, forward, sampling), visible in Nsight
timelines. Off unless ``METRALE_NVTX=1`` and CUDA is present: the disabled path is one attribute
test. Role of the reference's NVTX shim (``crates/gpu-sys`` nvtx bindings)."""
from __future__ import annotations

import os
from contextlib import contextmanager

_enabled = None


def enabled() -> bool:
    global _enabled
    if _enabled is None:
        _enabled = False
        if os.environ.get("METRALE_NVTX", "0") == "1":
            try:
                import torch
                _enabled = torch.cuda.is_available()
            except Exception:
                _enabled = False
    return _enabled


@contextmanager
def range(name: str):          # noqa: A001 - mirrors torch.cuda.nvtx.range
    if not enabled():
        yield
        return
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def mark(name: str) -> None:
    if enabled():
        import torch
        torch.cuda.nvtx.mark(name)
