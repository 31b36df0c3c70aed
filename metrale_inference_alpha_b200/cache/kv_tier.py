"""A second tier under the prefix cache: KV blocks the radix tree evicts go to host memory / files instead
of being lost, and a later request with the same prefix gets them back by a copy instead of a prefill.

``KvTierStore`` keeps fixed-size records (one record = one block of every cache layer, K and V) in a byte
store of the storage package (files with an optional pinned write-back host tier, or host memory), indexed
by the *chain digest* of the block: a hash over the namespace, every token of the prefix up to and including
the block. Capacity is bounded; the least recently used record is overwritten. The floating-point fields of a
record can go through a codec of ``cache/kv_codec.py`` (``nvfp4``: 76 bytes per 128-channel row; ``turbo4`` /
``turbo3`` / ``turbo2``: 68 / 52 / 36, against 256 for bf16). These encodings are lossy; they are applied on the way
into the tier and undone on the way back, the device pool keeps its own dtype.

``TieredRadixTree`` is the prefix tree with two hooks: ``evict`` writes a leaf's block to the store before the
block goes back to the allocator, and ``match`` continues past the last resident block while the store holds
the next chain digest — it allocates a block, restores the record into it and adopts it into the tree, so
the scheduler sees an ordinary (longer) prefix hit. Models with recurrent state are not tiered this way
(their prefix hits need state snapshots, which have their own tiers in ``cache/state_pool.py``).

Reference: the generic tiered cache and KV paging of ``crates/storage`` (``tier/``, ``kv_paging/``) under the
radix prefix cache of ``crates/cache``.
"""
from __future__ import annotations

import hashlib
from array import array
from collections import OrderedDict
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from .radix import PrefixMatch, RadixTree


def chain_digest(parent: bytes, key: Sequence[int], ns: Hashable = None) -> bytes:
    h = hashlib.blake2b(digest_size=16)
    h.update(parent if parent else repr(ns).encode())
    h.update(array("q", key).tobytes())
    return h.digest()


class KvTierStore:
    def __init__(self, kv, capacity_blocks: int, directory: Optional[str] = None, host_cache_blocks: int = 0,
                 direct_io: bool = False, codec: str = "raw"):
        from ..storage.backend import CascadeBackend, FileBackend, KvLayout, MemoryBackend, pinned_bytes
        if capacity_blocks <= 0:
            raise ValueError("the KV tier needs a positive capacity")
        from .kv_codec import make_codec
        self.kv, self.codec = kv, make_codec(codec)
        sample = kv.gather_blocks([0])
        self.fields = []                      # (name, dtype, shape, bytes in the record, packed as nvfp4)
        self.raw_bytes = 0
        for name, t in sorted(sample.items()):
            raw = t[0].numel() * t.element_size()
            self.raw_bytes += raw
            K = t.shape[-1]
            packed = self.codec.applies(t.dtype, K)
            n = (t[0].numel() // K) * self.codec.row_bytes(K, t.element_size()) if packed else raw
            self.fields.append((name, t.dtype, tuple(t.shape[1:]), n, packed))
        self.record_bytes = sum(f[3] for f in self.fields)
        layout = KvLayout(1, capacity_blocks, 1, 1, (self.record_bytes + 1) // 2, elem_bytes=1)
        backend = FileBackend(directory, layout, direct=direct_io) if directory else MemoryBackend(layout)
        if host_cache_blocks:
            backend = CascadeBackend(backend, host_cache_blocks)
        self.backend, self.layout = backend, layout
        self.capacity = capacity_blocks
        self.index: "OrderedDict[bytes, int]" = OrderedDict()          # digest -> record slot, least recently used first
        self.free = list(range(capacity_blocks - 1, -1, -1))
        self._buf = pinned_bytes(layout.block_bytes)
        self.stats = {"stored": 0, "restored": 0, "overwritten": 0, "bytes_out": 0, "bytes_in": 0}

    def has(self, digest: bytes) -> bool:
        return digest in self.index

    def put(self, digest: bytes, block: int) -> None:
        if digest in self.index:
            self.index.move_to_end(digest)
            return
        if not self.free:
            _, slot = self.index.popitem(last=False)
            self.stats["overwritten"] += 1
        else:
            slot = self.free.pop()
        data = self.kv.gather_blocks([block])
        off = 0
        for name, _, _, n, packed in self.fields:
            src = data[name][0].contiguous()
            if packed:
                src = self.codec.encode(src.reshape(-1, src.shape[-1])).contiguous()
            self._buf[off:off + n].copy_(src.view(torch.uint8).reshape(-1))
            off += n
        self.backend.write_block(0, slot, self._buf)
        self.index[digest] = slot
        self.stats["stored"] += 1
        self.stats["bytes_out"] += self.record_bytes

    def restore(self, digest: bytes, block: int) -> bool:
        slot = self.index.get(digest)
        if slot is None:
            return False
        self.index.move_to_end(digest)
        self.backend.read_block(0, slot, self._buf)
        data, off = {}, 0
        for name, dt, shape, n, packed in self.fields:
            rec = self._buf[off:off + n].clone()
            if packed:
                K = shape[-1]
                per_row = self.codec.row_bytes(K, 0)
                data[name] = self.codec.decode(rec.view(n // per_row, per_row), K).to(dt).view(1, *shape)
            else:
                data[name] = rec.view(dt).view(1, *shape)
            off += n
        self.kv.scatter_blocks([block], data)
        self.stats["restored"] += 1
        self.stats["bytes_in"] += self.record_bytes
        return True

    def close(self) -> None:
        self.backend.close()


class TieredRadixTree(RadixTree):
    def __init__(self, allocator, block_size: int, store: KvTierStore):
        super().__init__(allocator, block_size, needs_snapshot=False)
        self.store = store
        self.tier_hits = 0
        self.tier_hit_tokens = 0

    def _node_digest(self, node, ns) -> bytes:
        d = getattr(node, "chain", None)              # kept on the node itself: it lives exactly as long as the node
        if d is None:
            parent = b"" if node.parent is None or node.parent.parent is None else self._node_digest(node.parent, ns)
            d = node.chain = chain_digest(parent, node.key, ns)
        return d

    def _ns_of(self, node) -> Hashable:
        while node.parent is not None:
            node = node.parent
        for ns, root in self._roots.items():
            if root is node:
                return ns
        return None

    # ------------------------------------------------------------------ lookup: continue into the tier
    def match(self, tokens: Sequence[int], adapter: Hashable = None, max_tokens: Optional[int] = None) -> PrefixMatch:
        m = super().match(tokens, adapter, max_tokens)
        limit = len(tokens) - 1 if max_tokens is None else min(max_tokens, len(tokens) - 1)
        bs = self.block_size
        chunks = list(self._chunks(tokens))
        # the digest of the last resident block of the match
        node = self._root(adapter)
        for key in chunks[:len(m.blocks)]:
            node = node.children[key]
        digest = b"" if not m.blocks else self._node_digest(node, adapter)
        blocks = list(m.blocks)
        restored = 0
        while len(blocks) < len(chunks) and (len(blocks) + 1) * bs <= limit:
            nxt = chain_digest(digest, chunks[len(blocks)], adapter)
            if not self.store.has(nxt):
                break
            if self.alloc.num_free < 1 and self.evict(1) < 1:     # make room by demoting a colder block (never one of
                break                                              # this match: those carry the caller's reference)
            blk = self.alloc.alloc(1)[0]                      # the caller's reference
            if not self.store.restore(nxt, blk):
                self.alloc.free([blk])
                break
            blocks.append(blk)
            digest = nxt
            restored += 1
        if restored:
            self.insert(tokens[:len(blocks) * bs], blocks, adapter)       # the tree adopts the restored blocks
            self.tier_hits += 1
            self.tier_hit_tokens += restored * bs
            if not m.blocks:
                self.hits += 1
            self.hit_tokens += restored * bs
        return PrefixMatch(blocks, len(blocks) * bs, None)

    # ------------------------------------------------------------------ eviction: demote instead of drop
    def evict(self, num_blocks: int) -> int:
        freed = 0
        while freed < num_blocks:
            cands = [n for n in self._leaves() if self.alloc.refcount[n.block] == 1]
            if not cands:
                break
            cands.sort(key=lambda n: n.last_use)
            for n in cands:
                if freed >= num_blocks:
                    break
                self.store.put(self._node_digest(n, self._ns_of(n)), n.block)
                del n.parent.children[n.key]
                self.num_nodes -= 1
                freed += len(self.alloc.free([n.block]))
        return freed

    def stats(self) -> dict:
        s = super().stats()
        s.update({"tier_hits": self.tier_hits, "tier_hit_tokens": self.tier_hit_tokens, "tier_records": len(self.store.index),
                  **{f"tier_{k}": v for k, v in self.store.stats.items()}})
        return s
