"""Builds the host-side native runtime library (C++: block allocator, radix prefix index,
batch staging) next to this file. Pure g++, no CUDA. Safe to call repeatedly."""
from __future__ import annotations

import hashlib
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libmetrale_host.so"


def build(force: bool = False) -> Path:
    srcs = sorted(HERE.glob("*.cpp"))
    if not srcs:
        return LIB
    h = hashlib.sha256(b"".join(p.read_bytes() for p in srcs + sorted(HERE.glob("*.h")))).hexdigest()
    stamp = HERE / "build" / "stamp.txt"
    if not force and LIB.exists() and stamp.exists() and stamp.read_text() == h:
        return LIB
    stamp.parent.mkdir(exist_ok=True)
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-o", str(LIB)] + [str(s) for s in srcs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{r.stderr}")
    stamp.write_text(h)
    return LIB
