"""Radix-tree prefix cache over KV blocks, with a separate index of recurrent-state snapshots.

A node is one full block of ``block_size`` token ids; an edge is keyed by that tuple. The
tree holds one reference on every block it contains; a sequence that matches a prefix takes
its own references and keeps them until it finishes. Unreferenced leaves are evicted least
recently used first. Per-adapter roots keep LoRA variants apart. Models with recurrent layers
(gated-delta-net, Mamba2) can only reuse a prefix at a position where a state snapshot exists,
so matches are clipped to the deepest node carrying one.
Role of the reference's ``crates/cache/src/radix_tree.rs`` (+ ``radix_tree/snapshot*.rs``,
"Marconi" snapshots).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .block_pool import BlockAllocator


@dataclass
class _Node:
    key: Tuple[int, ...]
    block: int
    parent: Optional["_Node"]
    children: Dict[Tuple[int, ...], "_Node"] = field(default_factory=dict)
    last_use: int = 0
    snapshot: Optional[int] = None     # state-pool snapshot id valid *after* this block
    depth: int = 0                     # blocks from the root


@dataclass
class PrefixMatch:
    blocks: List[int]                  # matched blocks, already increfed for the caller
    tokens: int                        # matched token count (multiple of block_size)
    snapshot: Optional[int] = None     # snapshot to restore (recurrent models)


class RadixTree:
    def __init__(self, allocator: BlockAllocator, block_size: int, needs_snapshot: bool = False,
                 on_snapshot_evict=None):
        self.alloc = allocator
        self.block_size = block_size
        self.needs_snapshot = needs_snapshot
        self.on_snapshot_evict = on_snapshot_evict
        self.snapshot_ok = None              # optional predicate: is this snapshot handle still restorable (tiered pools)
        self._roots: Dict[Hashable, _Node] = {}
        self._clock = itertools.count(1)
        self.num_nodes = 0
        self.hits = 0
        self.queries = 0
        self.hit_tokens = 0

    def _root(self, adapter: Hashable) -> _Node:
        if adapter not in self._roots:
            self._roots[adapter] = _Node((), 0, None)
        return self._roots[adapter]

    def _chunks(self, tokens: Sequence[int]):
        bs = self.block_size
        for i in range(0, len(tokens) - len(tokens) % bs, bs):
            yield tuple(tokens[i:i + bs])

    # ------------------------------------------------------------------ lookup
    def match(self, tokens: Sequence[int], adapter: Hashable = None, max_tokens: Optional[int] = None
              ) -> PrefixMatch:
        """Longest cached prefix of `tokens` (whole blocks; never the full prompt, so at
        least one token is left to prefill). Takes a reference on every returned block."""
        self.queries += 1
        node = self._root(adapter)
        path: List[_Node] = []
        limit = len(tokens) - 1 if max_tokens is None else min(max_tokens, len(tokens) - 1)
        for key in self._chunks(tokens):
            if (len(path) + 1) * self.block_size > limit:
                break
            nxt = node.children.get(key)
            if nxt is None:
                break
            path.append(nxt)
            node = nxt
        snap = None
        if self.needs_snapshot:
            while path and (path[-1].snapshot is None
                            or (self.snapshot_ok is not None and not self.snapshot_ok(path[-1].snapshot))):
                path.pop()
            snap = path[-1].snapshot if path else None
        now = next(self._clock)
        for n in path:
            n.last_use = now
        blocks = [n.block for n in path]
        self.alloc.incref(blocks)
        if blocks:
            self.hits += 1
            self.hit_tokens += len(blocks) * self.block_size
        return PrefixMatch(blocks, len(blocks) * self.block_size, snap)

    # ------------------------------------------------------------------ insert
    def insert(self, tokens: Sequence[int], blocks: Sequence[int], adapter: Hashable = None,
               snapshots: Optional[Dict[int, int]] = None) -> int:
        """Publish the full blocks of a sequence. `blocks[i]` holds tokens [i*bs, (i+1)*bs).
        The tree takes its own reference on blocks it adopts; when a chunk is already present
        the existing block stays and the caller's duplicate is left alone. `snapshots` maps a
        token count (multiple of block_size) to a state snapshot id valid at that position.
        Returns the number of newly adopted blocks."""
        node = self._root(adapter)
        now = next(self._clock)
        adopted = 0
        for i, key in enumerate(self._chunks(tokens)):
            if i >= len(blocks):
                break
            nxt = node.children.get(key)
            if nxt is None:
                nxt = _Node(key, blocks[i], node, depth=node.depth + 1)
                node.children[key] = nxt
                self.alloc.incref([blocks[i]])
                self.num_nodes += 1
                adopted += 1
            nxt.last_use = now
            if snapshots:
                sid = snapshots.get((i + 1) * self.block_size)
                if sid is not None and nxt.snapshot is None:
                    nxt.snapshot = sid
            node = nxt
        return adopted

    # ------------------------------------------------------------------ eviction
    def _leaves(self):
        stack = list(self._roots.values())
        while stack:
            n = stack.pop()
            if n.children:
                stack.extend(n.children.values())
            elif n.parent is not None:
                yield n

    def evict(self, num_blocks: int) -> int:
        """Free up to `num_blocks` blocks held only by the tree, least recently used leaves
        first. Returns how many blocks went back to the allocator."""
        freed = 0
        while freed < num_blocks:
            cands = [n for n in self._leaves() if self.alloc.refcount[n.block] == 1]
            if not cands:
                break
            cands.sort(key=lambda n: n.last_use)
            for n in cands:
                if freed >= num_blocks:
                    break
                del n.parent.children[n.key]
                self.num_nodes -= 1
                if n.snapshot is not None and self.on_snapshot_evict:
                    self.on_snapshot_evict(n.snapshot)
                freed += len(self.alloc.free([n.block]))
        return freed

    def evictable_blocks(self) -> int:
        return sum(1 for n in self._all_nodes() if self.alloc.refcount[n.block] == 1)

    def _all_nodes(self):
        stack = list(self._roots.values())
        while stack:
            n = stack.pop()
            stack.extend(n.children.values())
            if n.parent is not None:
                yield n

    def clear(self) -> None:
        for n in list(self._all_nodes()):
            if n.snapshot is not None and self.on_snapshot_evict:
                self.on_snapshot_evict(n.snapshot)
            self.alloc.free([n.block])
        self._roots.clear()
        self.num_nodes = 0

    def stats(self) -> dict:
        return {"nodes": self.num_nodes, "queries": self.queries, "hits": self.hits,
                "hit_tokens": self.hit_tokens}
