"""High-speed swap: decode attention over KV blocks that live in files.

A long sequence's cold KV blocks are written to per-layer files (``offload_block``) and, at each
decode step, streamed back tile by tile through a small device scratch pool into the tiled attention
kernel (``attend_layer``), which keeps a running online-softmax state per (sequence, query head); an
optional last tile folds in the blocks that are still in the engine's own paged cache. A low-rank
predictor (K rows projected to ``r`` dims at offload time, the step's queries projected the same way)
scores every block per step; the scores only rank eviction victims of the scratch pool — attention
always reads every block, so the result does not depend on the predictor.

Overlap: the file reads of tile t + 1 are in flight in the I/O pool while tile t's host-to-device
copies and kernel are queued on the stream; staging buffers are recycled behind CUDA events.

Pieces: ``HighSpeedSwapConfig`` (range checks), ``DiskBlocks`` (id allocator: free list first, then
fresh ids, reference counts for shared prefixes), ``ScratchPool`` (slot <-> (layer, block) maps),
``EvictionPolicy`` ((score, last access) ascending over unpinned slots), ``Predictor``,
``TiledAttention`` and the ``HighSpeedSwap`` orchestrator with a per-thread installation slot through
which model code reaches it.

Reference: ``crates/storage/src/{high_speed_swap,config,scratch_pool,eviction,predictor,projection,
tiled_attention,model_dims}.rs``.
"""
from __future__ import annotations

import math
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import kernels as K
from .backend import CascadeBackend, FileBackend, KvLayout, MemoryBackend, StorageBackend, pinned_bytes


@dataclass
class ModelDims:
    num_layers: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    kv_dtype: torch.dtype = torch.bfloat16           # bf16, or float8_e4m3fn with per-layer scales

    @property
    def elem_bytes(self) -> int:
        return 1 if self.kv_dtype in (torch.float8_e4m3fn, torch.uint8) else 2


@dataclass
class HighSpeedSwapConfig:
    dir: Optional[str] = None            # None: host memory backend
    block_size: int = 16
    max_blocks_per_layer: int = 4096
    resident_blocks: int = 64            # scratch slots on the device
    tile_capacity: int = 16              # blocks per sequence per kernel launch
    rank: int = 32                       # predictor dims
    projection_seed: int = 0x5EED
    host_cache_blocks: int = 0           # > 0: pinned write-back cache in front of the files
    direct_io: bool = False
    io_workers: int = 8
    max_seqs: int = 8

    def validate(self, model: ModelDims) -> None:
        if model.num_q_heads % model.num_kv_heads:
            raise ValueError("num_q_heads must be a multiple of num_kv_heads")
        if model.num_q_heads // model.num_kv_heads > 8:
            raise ValueError("at most 8 query heads per kv head")
        if model.head_dim not in (128, 256):
            raise ValueError("head_dim must be 128 or 256")
        if not 1 <= self.rank <= 64:
            raise ValueError("rank must be in 1..64")
        for name in ("block_size", "max_blocks_per_layer", "resident_blocks", "tile_capacity", "max_seqs"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")
        if self.tile_capacity > self.resident_blocks:
            raise ValueError("tile_capacity cannot exceed resident_blocks")


class DiskBlocks:
    """Ids name the same block position in every layer's file."""

    def __init__(self, limit: int):
        self.limit, self.next_id = limit, 0
        self.free: List[int] = []
        self.refcount: Dict[int, int] = {}

    def alloc(self) -> int:
        if self.free:
            i = self.free.pop()
        elif self.next_id < self.limit:
            i, self.next_id = self.next_id, self.next_id + 1
        else:
            raise MemoryError(f"all {self.limit} disk blocks per layer are in use")
        self.refcount[i] = 1
        return i

    def retain(self, i: int) -> None:
        if self.refcount.get(i, 0) <= 0:
            raise KeyError(f"disk block {i} is not allocated")
        self.refcount[i] += 1

    def release(self, i: int) -> bool:
        n = self.refcount.get(i, 0)
        if n <= 0:
            raise KeyError(f"disk block {i} is not allocated")
        if n == 1:
            del self.refcount[i]
            self.free.append(i)
            return True
        self.refcount[i] = n - 1
        return False


class EvictionPolicy:
    def __init__(self):
        self.score: Dict[Tuple[int, int], float] = {}
        self.access: Dict[Tuple[int, int], int] = {}
        self.epoch = 0

    def tick(self) -> None:
        self.epoch += 1

    def touch(self, key) -> None:
        self.access[key] = self.epoch

    def record_score(self, key, s: float) -> None:
        self.score[key] = s

    def forget(self, key) -> None:
        self.score.pop(key, None)
        self.access.pop(key, None)

    def rank(self, keys: Sequence[Tuple[int, int]]) -> List[Tuple[int, int]]:
        """Eviction order: least important, then least recently used, first."""
        return sorted(keys, key=lambda k: (self.score.get(k, float("-inf")), self.access.get(k, -1), k))


class ScratchPool:
    """Device slots of one block each in the file layout: the K stripes of every kv head
    (``[tok][dim]`` rows, padded to the layout's group stride), then the V stripes."""

    def __init__(self, layout: KvLayout, slots: int, device, dtype: torch.dtype):
        self.layout, self.slots = layout, slots
        self.data = torch.zeros(slots, layout.block_bytes, dtype=torch.uint8, device=device)
        self.residents: List[Optional[Tuple[int, int]]] = [None] * slots
        self.lookup: Dict[Tuple[int, int], int] = {}
        self.free = list(range(slots - 1, -1, -1))
        self.dtype = dtype

    def strides(self) -> K.Strides:
        e = self.layout.elem_bytes
        return self.layout.block_bytes // e, self.layout.head_dim, self.layout.group_stride // e

    def pools(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(K view, V view) of the whole pool in elements; V starts kv_heads groups after K."""
        flat = self.data.view(-1)
        elems = flat.view(self.dtype) if self.dtype != torch.uint8 else flat
        return elems, elems[self.layout.kv_heads * self.layout.group_stride // self.layout.elem_bytes:]

    def slot_of(self, key) -> Optional[int]:
        return self.lookup.get(key)

    def place(self, key, slot: int) -> None:
        old = self.residents[slot]
        if old is not None:
            del self.lookup[old]
        self.residents[slot] = key
        self.lookup[key] = slot

    def drop(self, key) -> None:
        slot = self.lookup.pop(key, None)
        if slot is not None:
            self.residents[slot] = None
            self.free.append(slot)


def build_projection(head_dim: int, r: int, seed: int) -> torch.Tensor:
    """Fixed random projection with orthonormal columns (so projected dot products are unbiased up to
    the factor r / head_dim), drawn on the host from ``seed``."""
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(head_dim, r, generator=g, dtype=torch.float64))
    return (q * math.sqrt(head_dim / r)).to(torch.bfloat16)


class Predictor:
    def __init__(self, model: ModelDims, cfg: HighSpeedSwapConfig, device):
        self.P = build_projection(model.head_dim, cfg.rank, cfg.projection_seed).to(device)
        # per-token low-rank keys of every disk block: [layers, blocks, kv_heads, block, r]
        self.a_g = torch.zeros(model.num_layers, cfg.max_blocks_per_layer, model.num_kv_heads, cfg.block_size,
                               cfg.rank, dtype=torch.bfloat16, device=device)
        self.model, self.cfg = model, cfg

    def project_q(self, q: torch.Tensor) -> torch.Tensor:
        return K.project_rows(q, self.P)

    def project_block(self, layer: int, disk_id: int, k_pool, src_block: int, strides, k_scale: float = 1.0):
        dev = self.P.device
        K.project_blocks(k_pool, self.P, self.a_g[layer], torch.tensor([src_block], dtype=torch.int32, device=dev),
                         torch.tensor([disk_id], dtype=torch.int32, device=dev), Hkv=self.model.num_kv_heads,
                         block_size=self.cfg.block_size, strides=strides, k_scale=k_scale)

    def score(self, layer: int, q_lr, blocks, counts, last_valid=None) -> torch.Tensor:
        return K.predictor_score(q_lr, self.a_g[layer], blocks, counts, last_valid)


class TiledAttention:
    """``begin_step`` / ``step_tile`` ... / ``finalize`` around the running (m, l, o) state, allocated
    once for ``max_seqs`` sequences."""

    def __init__(self, model: ModelDims, max_seqs: int, device):
        self.model = model
        self.m, self.l, self.o = K.attn_state(max_seqs, model.num_q_heads, model.head_dim, device)
        self.n = 0

    def begin_step(self, num_seqs: int) -> None:
        if num_seqs > self.m.shape[0]:
            raise ValueError(f"{num_seqs} sequences exceed max_seqs {self.m.shape[0]}")
        self.n = num_seqs
        self.m[:num_seqs].fill_(float("-inf"))
        self.l[:num_seqs].zero_()
        self.o[:num_seqs].zero_()

    def step_tile(self, q, k_pool, v_pool, tile_blocks, tile_counts, *, block_size, strides, last_valid=None,
                  k_scale=1.0, v_scale=1.0, scale=None) -> None:
        n = self.n
        K.kv_tile_attn(q, k_pool, v_pool, tile_blocks, tile_counts, (self.m[:n], self.l[:n], self.o[:n]),
                       Hkv=self.model.num_kv_heads, block_size=block_size, strides=strides, last_valid=last_valid,
                       scale=scale, k_scale=k_scale, v_scale=v_scale)

    def finalize(self) -> torch.Tensor:
        return K.attn_finalize(self.l[:self.n], self.o[:self.n])


@dataclass
class ResidentTail:
    """Blocks of the step that are still in the engine's paged cache (folded in as the last tile)."""
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    block_table: torch.Tensor          # [S, cap] int32
    counts: torch.Tensor               # [S] int32
    last_valid: Optional[torch.Tensor]
    strides: K.Strides


_local = threading.local()


class HighSpeedSwap:
    def __init__(self, cfg: HighSpeedSwapConfig, model: ModelDims, device="cpu", backend: Optional[StorageBackend] = None):
        cfg.validate(model)
        self.cfg, self.model, self.device = cfg, model, torch.device(device)
        self.layout = KvLayout(model.num_layers, cfg.max_blocks_per_layer, cfg.block_size, model.num_kv_heads,
                               model.head_dim, model.elem_bytes)
        if backend is None:
            backend = (FileBackend(cfg.dir, self.layout, direct=cfg.direct_io, workers=cfg.io_workers)
                       if cfg.dir else MemoryBackend(self.layout))
            if cfg.host_cache_blocks:
                backend = CascadeBackend(backend, cfg.host_cache_blocks)
        self.backend = backend
        store = torch.uint8 if model.elem_bytes == 1 else model.kv_dtype
        self.pool = ScratchPool(self.layout, cfg.resident_blocks, self.device, store)
        self.predictor = Predictor(model, cfg, self.device)
        self.attn = TiledAttention(model, cfg.max_seqs, self.device)
        self.eviction = EvictionPolicy()
        self.disk = DiskBlocks(cfg.max_blocks_per_layer)
        self._staging = [pinned_bytes(self.layout.block_bytes) for _ in range(2 * cfg.resident_blocks)]
        self._staging_ev: List[Optional[torch.cuda.Event]] = [None] * len(self._staging)
        self._stage_i = 0
        self.kv_scales: Dict[int, Tuple[float, float]] = {}
        self.stats = {"offloaded": 0, "tiles": 0, "slot_hits": 0, "slot_misses": 0, "evictions": 0}

    # ------------------------------------------------------------------ per-thread installation
    def install_local(self) -> None:
        _local.hss = self

    @staticmethod
    def with_local(fn):
        hss = getattr(_local, "hss", None)
        return None if hss is None else fn(hss)

    @staticmethod
    def uninstall_local() -> None:
        _local.hss = None

    # ------------------------------------------------------------------ offload
    def alloc_disk_block(self) -> int:
        return self.disk.alloc()

    def release_disk_block(self, disk_id: int) -> None:
        if self.disk.release(disk_id):
            for layer in range(self.model.num_layers):
                self.pool.drop((layer, disk_id))
                self.eviction.forget((layer, disk_id))

    def set_kv_scales(self, layer: int, k_scale: float, v_scale: float) -> None:
        self.kv_scales[layer] = (float(k_scale), float(v_scale))

    def _next_staging(self) -> Tuple[int, torch.Tensor]:
        i = self._stage_i
        self._stage_i = (i + 1) % len(self._staging)
        ev = self._staging_ev[i]
        if ev is not None:
            ev.synchronize()
            self._staging_ev[i] = None
        return i, self._staging[i]

    def offload_block(self, layer: int, disk_id: int, k_block: torch.Tensor, v_block: torch.Tensor) -> None:
        """``k_block`` / ``v_block`` [block, kv_heads, D] (one block of the engine's paged cache, any
        device): written to the layer file as per-head stripes; the block's low-rank keys are stored
        for the predictor."""
        L = self.layout
        if tuple(k_block.shape) != (L.block_size, L.kv_heads, L.head_dim) or k_block.shape != v_block.shape:
            raise ValueError(f"block must be [{L.block_size}, {L.kv_heads}, {L.head_dim}]")
        i, buf = self._next_staging()
        buf.zero_()
        for kind, blk in ((0, k_block), (1, v_block)):
            stripes = blk.permute(1, 0, 2).contiguous()                      # [kv_head, tok, D]
            raw = stripes.view(torch.uint8) if stripes.dtype != torch.uint8 else stripes
            raw = raw.reshape(L.kv_heads, L.group_payload).cpu()
            for h in range(L.kv_heads):
                off = L.file_offset(0, kind, h)
                buf[off:off + L.group_payload].copy_(raw[h])
        self.backend.write_block(layer, disk_id, buf)
        ks = self.kv_scales.get(layer, (1.0, 1.0))[0]
        kp = k_block.to(self.device).contiguous()
        kp = kp.view(torch.uint8) if self.model.elem_bytes == 1 else kp
        self.predictor.project_block(layer, disk_id, kp, 0, K.paged_strides(L.block_size, L.kv_heads, L.head_dim), ks)
        self.stats["offloaded"] += 1

    # ------------------------------------------------------------------ attend
    def _victim(self, pinned: set) -> int:
        if self.pool.free:
            return self.pool.free.pop()
        cands = [k for k in self.pool.lookup if k not in pinned]
        if not cands:
            raise RuntimeError("every scratch slot is pinned by the current tile")
        key = self.eviction.rank(cands)[0]
        slot = self.pool.lookup[key]
        self.stats["evictions"] += 1
        return slot

    def _issue(self, layer: int, wanted: List[int]) -> list:
        """Start the file reads of the blocks of a tile that are not in the scratch pool."""
        missing = [d for d in wanted if self.pool.slot_of((layer, d)) is None]
        stage = [self._next_staging() for _ in missing]
        futs = self.backend.read_blocks_async(layer, missing, [b for _, b in stage]) if missing else []
        return [(d, si, buf, f) for d, (si, buf), f in zip(missing, stage, futs)]

    def _land(self, layer: int, wanted: List[int], pending: list) -> Dict[int, int]:
        """Make a tile resident: wait for its reads, pick victims (never a block of this tile) and
        queue the host-to-device copies on the current stream. Returns disk id -> slot."""
        pinned = {(layer, d) for d in wanted}
        for d in wanted:
            self.eviction.touch((layer, d))
        for d, si, buf, f in pending:
            f.result()
            if self.pool.slot_of((layer, d)) is None:
                slot = self._victim(pinned)
                self.pool.place((layer, d), slot)
                self.pool.data[slot].copy_(buf, non_blocking=True)
                if self.device.type == "cuda":
                    ev = torch.cuda.Event()
                    ev.record()
                    self._staging_ev[si] = ev
            self.stats["slot_misses"] += 1
        self.stats["slot_hits"] += len(wanted) - len(pending)
        return {d: self.pool.lookup[(layer, d)] for d in wanted}

    def prefetch(self, layer: int, disk_ids: Sequence[int]) -> None:
        """Bring the first blocks the next step will want into the scratch pool ahead of it."""
        ids = list(dict.fromkeys(disk_ids))[: self.cfg.tile_capacity]
        if ids:
            self._land(layer, ids, self._issue(layer, ids))

    def attend_layer(self, layer: int, q: torch.Tensor, seq_blocks: Sequence[Sequence[int]],
                     last_valid: Optional[Sequence[int]] = None, tail: Optional[ResidentTail] = None,
                     scale: Optional[float] = None) -> torch.Tensor:
        """Decode attention of ``q`` [S, Hq, D] (bf16) over each sequence's offloaded blocks
        ``seq_blocks[s]`` (disk ids in order; ``last_valid[s]`` token slots are used in the last one)
        plus the optional device-resident ``tail``. Returns bf16 [S, Hq, D]."""
        S = q.shape[0]
        cfg, dev = self.cfg, self.device
        self.eviction.tick()
        self.attn.begin_step(S)
        ks, vs = self.kv_scales.get(layer, (1.0, 1.0))
        n_max = max((len(b) for b in seq_blocks), default=0)
        if n_max:
            # predictor: rank blocks for eviction (never for skipping)
            tbl = torch.zeros(S, n_max, dtype=torch.int32)
            for s, b in enumerate(seq_blocks):
                tbl[s, :len(b)] = torch.tensor(list(b), dtype=torch.int32)
            cnt = torch.tensor([len(b) for b in seq_blocks], dtype=torch.int32)
            scores = self.predictor.score(layer, self.predictor.project_q(q), tbl.to(dev), cnt.to(dev)).cpu()
            best: Dict[Tuple[int, int], float] = {}
            for s, b in enumerate(seq_blocks):
                for j, d in enumerate(b):
                    best[(layer, d)] = max(best.get((layer, d), float("-inf")), float(scores[s, j]))
            for key, v in best.items():
                self.eviction.record_score(key, v)
        cap = max(1, min(cfg.tile_capacity, cfg.resident_blocks // max(S, 1)))
        k_pool, v_pool = self.pool.pools()
        strides = self.pool.strides()
        tiles = [list(dict.fromkeys(d for b in seq_blocks for d in b[t0:t0 + cap])) for t0 in range(0, n_max, cap)]
        pending = self._issue(layer, tiles[0]) if tiles else []
        for i, wanted in enumerate(tiles):
            t0 = i * cap
            slots = self._land(layer, wanted, pending)
            # the next tile's reads run in the I/O pool while this tile's copies and kernel are queued
            pending = self._issue(layer, tiles[i + 1]) if i + 1 < len(tiles) else []
            tb = torch.zeros(S, cap, dtype=torch.int32)
            tc = torch.zeros(S, dtype=torch.int32)
            lv = torch.full((S,), cfg.block_size, dtype=torch.int32)
            for s, b in enumerate(seq_blocks):
                part = b[t0:t0 + cap]
                tc[s] = len(part)
                for j, d in enumerate(part):
                    tb[s, j] = slots[d]
                if last_valid is not None and part and t0 + cap >= len(b):
                    lv[s] = last_valid[s]
            self.attn.step_tile(q, k_pool, v_pool, tb.to(dev), tc.to(dev), block_size=cfg.block_size, strides=strides,
                                last_valid=lv.to(dev), k_scale=ks, v_scale=vs, scale=scale)
            self.stats["tiles"] += 1
        if tail is not None:
            self.attn.step_tile(q, tail.k_pool, tail.v_pool, tail.block_table, tail.counts, block_size=cfg.block_size,
                                strides=tail.strides, last_valid=tail.last_valid, k_scale=ks, v_scale=vs, scale=scale)
            self.stats["tiles"] += 1
        return self.attn.finalize()

    def close(self) -> None:
        self.backend.close()
