"""Storage capability probe: what the scratch directory can do and which backend to use.

Checks whether ``O_DIRECT`` opens work there, whether a GPUDirect Storage stack (libcufile + the
nvidia-fs module) is present, and times sequential block reads and writes through ``FileBackend``
(buffered, and direct when available); ``decide`` turns the results into a recommendation. A
benchmark that fails is recorded with its error and left out of the decision.

Reference: ``crates/storage/src/{probe,bench}.rs``.
"""
from __future__ import annotations

import ctypes.util
import os
import tempfile
import time
from typing import Dict, Optional

import torch

from .backend import FileBackend, KvLayout, pinned_bytes


def _bench(root: str, direct: bool, blocks: int, layout: KvLayout) -> Dict[str, float]:
    be = FileBackend(root, layout, direct=direct, workers=8)
    try:
        if direct and not be.direct:
            raise OSError("O_DIRECT refused by the filesystem")
        bufs = [pinned_bytes(layout.block_bytes) for _ in range(min(blocks, 16))]
        for b in bufs:
            b.random_(0, 255)
        t0 = time.perf_counter()
        for i in range(blocks):
            be.write_block(0, i, bufs[i % len(bufs)])
        be.flush()
        t1 = time.perf_counter()
        for i0 in range(0, blocks, len(bufs)):
            ids = list(range(i0, min(blocks, i0 + len(bufs))))
            for f in be.read_blocks_async(0, ids, bufs[:len(ids)]):
                f.result()
        t2 = time.perf_counter()
        n = blocks * layout.block_bytes
        return {"write_gbs": n / (t1 - t0) / 1e9, "read_gbs": n / (t2 - t1) / 1e9}
    finally:
        be.close()


def decide(report: dict) -> str:
    """``cufile`` is never recommended here (no binding to it exists in this tree); direct I/O wins
    when it works and reads at least as fast as the page cache path, else buffered files; with no
    usable directory at all, host memory."""
    if not report.get("dir_writable"):
        return "memory"
    d, b = report.get("direct"), report.get("buffered")
    if d and "read_gbs" in d and (not b or "read_gbs" not in b or d["read_gbs"] >= 0.8 * b["read_gbs"]):
        return "file-direct"
    return "file" if b and "read_gbs" in b else "memory"


def run_probe(root: Optional[str] = None, *, blocks: int = 64, block_kib: int = 256) -> dict:
    own = root is None
    root = root or tempfile.mkdtemp(prefix="metrale_probe_")
    rep: dict = {"dir": root, "o_direct_flag": hasattr(os, "O_DIRECT"),
                 "libcufile": ctypes.util.find_library("cufile") is not None,
                 "nvidia_fs_module": os.path.exists("/proc/driver/nvidia-fs"),
                 "pinned_host_memory": torch.cuda.is_available()}
    try:
        os.makedirs(root, exist_ok=True)
        rep["dir_writable"] = os.access(root, os.W_OK)
    except OSError as e:
        rep["dir_writable"], rep["dir_error"] = False, str(e)
    # one kv head of block_kib KiB per K / V stripe
    layout = KvLayout(1, blocks, block_kib * 1024 // (2 * 128 * 2), 1, 128)
    if rep["dir_writable"]:
        for name, direct in (("buffered", False), ("direct", True)):
            sub = os.path.join(root, name)
            try:
                rep[name] = _bench(sub, direct, blocks, layout)
            except Exception as e:             # recorded, not fatal
                rep[name] = {"error": f"{type(e).__name__}: {e}"}
            finally:
                p = layout.layer_path(sub, 0)
                if os.path.exists(p):
                    os.remove(p)
                if os.path.isdir(sub):
                    os.rmdir(sub)
    rep["recommendation"] = decide(rep)
    if own and os.path.isdir(root):
        try:
            os.rmdir(root)
        except OSError:
            pass
    return rep
