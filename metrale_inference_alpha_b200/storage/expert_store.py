"""MoE expert streaming: expert weights live in an on-disk store and are paged into a device arena
of a few slots, so a model whose experts do not fit in device memory still serves.

Store format. One file per MoE layer, ``experts_00000.bin``, of ``num_experts`` records at one stride
(the whole store shares it). A record is a fixed 64-byte header (magic, version, layer, expert,
payload bytes, four fp32 scalars) followed by the expert's sub-buffers in a fixed order — for each of
the gate/up and the down projection: packed weights, scales, per-row global scales — every sub-buffer
at a multiple of ``sub_align``, the record padded to a multiple of the filesystem block.
``manifest.json`` holds the version, the sub-buffer table and the record stride; a reader refuses a
manifest of another version and a record whose header names another (layer, expert).

Arena. ``PagedExperts`` owns one stacked weight pair of ``slots`` experts (the layout the grouped GEMM
reads) shared by all layers. ``waves(layer, idx)`` makes the experts a step routes to resident
(CLOCK / second-chance eviction; the experts of the current call are pinned), and returns the routing
ids rewritten to slot numbers; ids that are not resident in this wave are rewritten to -1, which the
expert sort drops, so a step that touches more experts than there are slots runs in several waves
whose outputs add up.

Reference: ``crates/storage/src/{expert,expert_pack,expert_pack_fs,expert_tier,expert_arena}.rs``.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

MAGIC = b"MBXP"
VERSION = 1
HEADER = struct.Struct("<4sIIIQ4f28x")          # 64 bytes
_DT = {"uint8": torch.uint8, "bfloat16": torch.bfloat16, "float32": torch.float32}


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass(frozen=True)
class SubBuffer:
    name: str           # e.g. "gate_up.data"
    dtype: str
    shape: Tuple[int, ...]
    offset: int         # from the start of the record
    nbytes: int


@dataclass
class RecordSpec:
    subs: List[SubBuffer]
    raw_bytes: int
    record_stride: int
    fmt: Tuple[str, str]                         # serving formats of (gate_up, down)
    dims: Tuple[int, int, int, int]              # gate_up N, K; down N, K
    interleaved: bool
    sub_align: int = 256
    fs_block: int = 4096

    @staticmethod
    def of(ffn, sub_align: int = 256, fs_block: int = 4096) -> "RecordSpec":
        subs, off = [], HEADER.size
        for part, w in (("gate_up", ffn.gate_up), ("down", ffn.down)):
            for field in ("data", "scale", "row_gscale"):
                t = getattr(w, field)
                if t is None:
                    continue
                off = _round_up(off, sub_align)
                n = t.numel() * t.element_size()
                subs.append(SubBuffer(f"{part}.{field}", str(t.dtype).replace("torch.", ""), tuple(t.shape), off, n))
                off += n
        return RecordSpec(subs, off, _round_up(off, fs_block), (ffn.gate_up.fmt, ffn.down.fmt),
                          (ffn.gate_up.N, ffn.gate_up.K, ffn.down.N, ffn.down.K), bool(ffn.interleaved),
                          sub_align, fs_block)

    def to_json(self) -> dict:
        return {"subs": [[s.name, s.dtype, list(s.shape), s.offset, s.nbytes] for s in self.subs],
                "raw_bytes": self.raw_bytes, "record_stride": self.record_stride, "fmt": list(self.fmt),
                "dims": list(self.dims), "interleaved": self.interleaved, "sub_align": self.sub_align,
                "fs_block": self.fs_block}

    @staticmethod
    def from_json(d: dict) -> "RecordSpec":
        subs = [SubBuffer(n, dt, tuple(sh), off, nb) for n, dt, sh, off, nb in d["subs"]]
        spec = RecordSpec(subs, d["raw_bytes"], d["record_stride"], tuple(d["fmt"]), tuple(d["dims"]),
                          d["interleaved"], d["sub_align"], d["fs_block"])
        spec.check()
        return spec

    def check(self) -> None:
        end = HEADER.size
        for s in self.subs:
            if s.offset % self.sub_align or s.offset < end:
                raise ValueError(f"sub-buffer {s.name} is misaligned or overlaps its predecessor")
            end = s.offset + s.nbytes
        if end > self.raw_bytes or self.record_stride % self.fs_block or self.record_stride < self.raw_bytes:
            raise ValueError("record geometry is inconsistent")


def pack_record(spec: RecordSpec, layer: int, expert: int, ffn) -> torch.Tensor:
    """One record in memory (uint8 [record_stride])."""
    buf = torch.zeros(spec.record_stride, dtype=torch.uint8)
    HEADER.pack_into(memoryview(buf.numpy()), 0, MAGIC, VERSION, layer, expert, spec.raw_bytes,
                     float(ffn.gate_up.gscale), float(ffn.down.gscale), float(ffn.down_in_scale), 0.0)
    for s in spec.subs:
        part, field = s.name.split(".")
        t = getattr(getattr(ffn, part), field).detach().cpu().contiguous()
        if tuple(t.shape) != s.shape:
            raise ValueError(f"{s.name}: shape {tuple(t.shape)} differs from the store's {s.shape}")
        buf[s.offset:s.offset + s.nbytes].copy_(t.view(torch.uint8).reshape(-1))
    return buf


def unpack_record(spec: RecordSpec, buf: torch.Tensor, layer: int, expert: int):
    """Views of a record's sub-buffers + its scalars; raises on a foreign or damaged header."""
    magic, ver, lay, exp, raw, g_gu, g_dn, d_in, _ = HEADER.unpack_from(memoryview(buf[:HEADER.size].numpy()), 0)
    if magic != MAGIC or ver != VERSION:
        raise ValueError("not an expert record of this version")
    if (lay, exp) != (layer, expert):
        raise ValueError(f"record holds expert ({lay}, {exp}), wanted ({layer}, {expert})")
    if raw != spec.raw_bytes:
        raise ValueError("record length differs from the manifest")
    views = {s.name: buf[s.offset:s.offset + s.nbytes].view(_DT[s.dtype]).view(s.shape) for s in spec.subs}
    return views, {"gate_up.gscale": g_gu, "down.gscale": g_dn, "down_in_scale": d_in}


def write_store(root: str, layers: Sequence[Sequence[object]]) -> RecordSpec:
    """``layers[l][e]`` = the FfnW of expert e of MoE layer l (all of one geometry)."""
    os.makedirs(root, exist_ok=True)
    spec = RecordSpec.of(layers[0][0])
    for li, experts in enumerate(layers):
        with open(os.path.join(root, f"experts_{li:05d}.bin"), "wb") as f:
            for ei, ffn in enumerate(experts):
                f.write(memoryview(pack_record(spec, li, ei, ffn).numpy()))
    manifest = {"version": VERSION, "num_layers": len(layers), "num_experts": len(layers[0]), "record": spec.to_json()}
    tmp = os.path.join(root, "manifest.json.tmp")
    with open(tmp, "w") as f:
        json.dump(manifest, f)
    os.replace(tmp, os.path.join(root, "manifest.json"))          # published last
    return spec


class ExpertFileReader:
    def __init__(self, root: str):
        with open(os.path.join(root, "manifest.json")) as f:
            m = json.load(f)
        if m.get("version") != VERSION:
            raise ValueError(f"expert store version {m.get('version')} is not {VERSION}")
        self.num_layers, self.num_experts = m["num_layers"], m["num_experts"]
        self.spec = RecordSpec.from_json(m["record"])
        self._fds = []
        for li in range(self.num_layers):
            path = os.path.join(root, f"experts_{li:05d}.bin")
            fd = os.open(path, os.O_RDONLY)
            if os.fstat(fd).st_size < self.num_experts * self.spec.record_stride:
                os.close(fd)
                raise ValueError(f"{path} is shorter than {self.num_experts} records")
            self._fds.append(fd)
        self.reads = 0

    def read_record(self, layer: int, expert: int, buf: torch.Tensor) -> None:
        if not (0 <= layer < self.num_layers and 0 <= expert < self.num_experts):
            raise IndexError(f"expert ({layer}, {expert}) outside the store")
        n = os.preadv(self._fds[layer], [memoryview(buf[:self.spec.record_stride].numpy())],
                      expert * self.spec.record_stride)
        if n != self.spec.record_stride:
            raise IOError("short read of an expert record")
        self.reads += 1

    def close(self) -> None:
        for fd in self._fds:
            os.close(fd)
        self._fds = []


class PagedExperts:
    def __init__(self, reader: ExpertFileReader, slots: int, device="cpu"):
        from ..ops import QuantWeight
        from ..ops.moe import GroupedExperts
        if slots <= 0:
            raise ValueError("the arena needs at least one slot")
        self.reader, self.slots, self.device = reader, slots, torch.device(device)
        spec = reader.spec
        self.spec = spec
        if "fp8_block" in spec.fmt and (spec.dims[0] % 128 or spec.dims[2] % 128):
            raise ValueError("block-scaled experts must have a multiple of 128 rows to share a stack")
        stacks = {}
        for part, fmt, N, Kd in (("gate_up", spec.fmt[0], spec.dims[0], spec.dims[1]),
                                 ("down", spec.fmt[1], spec.dims[2], spec.dims[3])):
            t = {}
            for s in spec.subs:
                p, field = s.name.split(".")
                if p == part:
                    t[field] = torch.zeros((slots * s.shape[0],) + s.shape[1:], dtype=_DT[s.dtype], device=self.device)
            w = QuantWeight(fmt, slots * N, Kd, t["data"], t.get("scale"))
            if fmt == "nvfp4":
                # every slot keeps its own global scale as a per-row scale of the stack
                w.row_gscale = t.get("row_gscale")
                if w.row_gscale is None:
                    w.row_gscale = torch.ones(slots * N, dtype=torch.float32, device=self.device)
                w.gscale = 1.0
                if self.device.type == "cuda":
                    if N % 128:
                        raise ValueError("NVFP4 experts must have a multiple of 128 rows to be paged")
                    w.prepare_cuda()
            stacks[part] = w
        self.grouped = GroupedExperts(stacks["gate_up"], stacks["down"], slots, spec.dims[0], spec.dims[2],
                                      spec.interleaved)
        self.resident: List[Optional[Tuple[int, int]]] = [None] * slots
        self.lookup: Dict[Tuple[int, int], int] = {}
        self.ref_bit = [False] * slots
        self.hand = 0
        self._staging = torch.empty(spec.record_stride, dtype=torch.uint8,
                                    pin_memory=torch.cuda.is_available() and self.device.type == "cuda")
        self.down_in_scale: Dict[Tuple[int, int], float] = {}
        self.stats = {"hits": 0, "loads": 0, "evictions": 0, "waves": 0}

    # ------------------------------------------------------------------ residency
    def _victim(self, pinned: set) -> int:
        for _ in range(2 * self.slots + 1):
            s = self.hand
            self.hand = (self.hand + 1) % self.slots
            key = self.resident[s]
            if key is None:
                return s
            if key in pinned:
                continue
            if self.ref_bit[s]:
                self.ref_bit[s] = False          # second chance
                continue
            del self.lookup[key]
            self.resident[s] = None
            self.stats["evictions"] += 1
            return s
        raise RuntimeError("every arena slot is pinned")

    def _load(self, layer: int, expert: int, slot: int) -> None:
        self.reader.read_record(layer, expert, self._staging)
        views, scal = unpack_record(self.spec, self._staging, layer, expert)
        for part, w, N in (("gate_up", self.grouped.gate_up, self.spec.dims[0]), ("down", self.grouped.down, self.spec.dims[2])):
            for field in ("data", "scale", "row_gscale"):
                v = views.get(f"{part}.{field}")
                if v is None:
                    continue
                dst = getattr(w, field)
                rows = v.shape[0]
                dst[slot * rows:(slot + 1) * rows].copy_(v, non_blocking=False)
            if w.fmt == "nvfp4":
                g = scal[f"{part}.gscale"]
                if f"{part}.row_gscale" in views:
                    w.row_gscale[slot * N:(slot + 1) * N].mul_(g)
                else:
                    w.row_gscale[slot * N:(slot + 1) * N].fill_(g)
                if self.device.type == "cuda":
                    self._retile(w, slot, N)
        self.down_in_scale[(layer, expert)] = scal["down_in_scale"]
        self.resident[slot] = (layer, expert)
        self.lookup[(layer, expert)] = slot
        self.ref_bit[slot] = True
        self.stats["loads"] += 1

    @staticmethod
    def _retile(w, slot: int, N: int) -> None:
        """Rebuild the tiled scale-factor copy of one slot's rows (whole 128-row tiles by construction)."""
        from ..ops import _count, _native, _ptr, _stream
        kblocks = w.K // 16
        tile_bytes = (N // 128) * w.sf_k64 * 512
        src = w.scale[slot * N:(slot + 1) * N]
        dst = w.sf_tiled[slot * tile_bytes:(slot + 1) * tile_bytes]
        _native.check(_native.lib().mb_sf_repack(_ptr(src), _ptr(dst), N, kblocks, w.sf_k64, _stream()), "sf_repack")
        _count()

    def waves(self, layer: int, idx: torch.Tensor):
        """Yield the routing ids rewritten to arena slots (int32, -1 = not in this wave), one tensor per
        wave of at most ``slots`` distinct experts; all experts of a wave are resident when it is
        yielded."""
        experts = [int(e) for e in torch.unique(idx).tolist() if e >= 0]
        for w0 in range(0, len(experts), self.slots):
            wave = experts[w0:w0 + self.slots]
            pinned = {(layer, e) for e in wave}
            for e in wave:
                s = self.lookup.get((layer, e))
                if s is None:
                    self._load(layer, e, self._victim(pinned))
                else:
                    self.ref_bit[s] = True
                    self.stats["hits"] += 1
            lut = torch.full((self.reader.num_experts + 1,), -1, dtype=torch.int32)
            for e in wave:
                lut[e] = self.lookup[(layer, e)]
            self.stats["waves"] += 1
            yield lut.to(idx.device)[idx.long().clamp_(min=-1)]

    def slot_ffn(self, slot: int):
        """FfnW view of one slot (the per-expert path of CPU tensors)."""
        from ..ops import QuantWeight
        from ..weights.loader import FfnW
        parts = []
        for w, N in ((self.grouped.gate_up, self.spec.dims[0]), (self.grouped.down, self.spec.dims[2])):
            rows = slice(slot * N, (slot + 1) * N)
            scale = None
            if w.scale is not None:
                per = w.scale.shape[0] // self.slots
                scale = w.scale[slot * per:(slot + 1) * per]
            q = QuantWeight(w.fmt, N, w.K, w.data[rows], scale)
            if w.row_gscale is not None:
                q.row_gscale = w.row_gscale[rows]
            parts.append(q)
        key = self.resident[slot]
        return FfnW(parts[0], parts[1], self.spec.interleaved, self.down_in_scale.get(key, 0.0))


def enable_expert_paging(model_w, root: str, slots: int, device) -> PagedExperts:
    """Move the routed experts of every MoE layer of a loaded model into an expert store under
    ``root`` (written from the loaded weights when no manifest is there yet) and replace them by one
    shared arena of ``slots`` experts. Shared experts, routers and everything else stay resident."""
    moe_layers = [L for L in model_w.layers if getattr(L, "ffn_kind", "") == "moe"]
    if not moe_layers:
        raise ValueError("the model has no MoE layers")
    if any(L.ffn.expert_lo != 0 for L in moe_layers):
        raise ValueError("expert paging and expert parallelism are separate ways to hold the experts: use one")
    if not os.path.exists(os.path.join(root, "manifest.json")):
        write_store(root, [L.ffn.experts for L in moe_layers])
    paged = PagedExperts(ExpertFileReader(root), slots, device)
    if paged.reader.num_layers != len(moe_layers):
        raise ValueError(f"the store holds {paged.reader.num_layers} MoE layers, the model has {len(moe_layers)}")
    for i, L in enumerate(moe_layers):
        w = L.ffn
        w.experts, w.grouped, w.router_ext = [], None, None
        w.paged, w.paged_layer = paged, i
    return paged
