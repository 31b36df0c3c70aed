"""Checkpoint reader on the C++ parallel file reader: parses the safetensors headers itself
(8-byte little-endian header length, JSON of ``{name: {dtype, shape, data_offsets}}``), reads
tensor bytes with a pool of ``pread`` threads (optionally O_DIRECT) straight into pinned host
buffers, and issues one asynchronous host-to-device copy per tensor, so the file reads of the
next tensors overlap the copies of the previous ones. ``prefetch(names)`` reads a whole group
(one layer) in a single call. Role of the reference's fast weight loader
(``crates/model-weights/src/fast_weights/mod.rs``; header math ``crates/core/src/safetensors.rs``).
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Dict, Iterable, List, Tuple

import torch

from .. import native
from .source import SafetensorsSource

_DT = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
       "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
       "BOOL": torch.bool, "F8_E4M3": torch.uint8, "F8_E5M2": torch.uint8, "F8_E8M0": torch.uint8}


def read_header(path: Path) -> Tuple[Dict[str, dict], int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > 256 << 20:
            raise ValueError(f"{path}: implausible safetensors header of {n} bytes")
        meta = json.loads(f.read(n))
    meta.pop("__metadata__", None)
    return meta, 8 + n


class FastSafetensorsSource(SafetensorsSource):
    def __init__(self, path, device="cpu", threads: int = 8, direct: bool = False):
        super().__init__(path, device="cpu")
        self.target = torch.device(device)
        self.threads, self.direct = threads, direct
        self._meta: Dict[Path, Tuple[Dict[str, dict], int]] = {}
        self._ready: Dict[str, torch.Tensor] = {}
        self.bytes_read = 0

    def _entry(self, name: str):
        f = self._index[name]
        if f not in self._meta:
            self._meta[f] = read_header(f)
        meta, base = self._meta[f]
        e = meta[name]
        b, end = e["data_offsets"]
        return f, e, base + b, end - b

    def prefetch(self, names: Iterable[str]) -> None:
        """Read every named tensor that is not yet staged; one reader call per shard file."""
        by_file: Dict[Path, List[Tuple[str, dict, int, int]]] = {}
        for n in names:
            if n in self._ready or n not in self._index:
                continue
            f, e, off, size = self._entry(n)
            by_file.setdefault(f, []).append((n, e, off, size))
        pin = self.target.type == "cuda"
        for f, items in by_file.items():
            bufs = [torch.empty(max(1, size), dtype=torch.uint8, pin_memory=pin) for _, _, _, size in items]
            self.bytes_read += native.read_ranges(str(f), [o for _, _, o, _ in items], [s for _, _, _, s in items],
                                                  [b.data_ptr() for b in bufs], self.threads, self.direct)
            for (n, e, _, size), b in zip(items, bufs):
                t = b[:size].view(_DT[e["dtype"]]).reshape(e["shape"])
                self._ready[n] = t.to(self.target, non_blocking=True) if pin else t

    def get(self, name):
        if name not in self._ready:
            self.prefetch([name])
        return self._ready.pop(name)


def open_source(path, device="cpu"):
    """The fast reader when the host runtime library is built, else the safetensors package."""
    if native.available():
        return FastSafetensorsSource(path, device=device)
    return SafetensorsSource(path, device=device)
