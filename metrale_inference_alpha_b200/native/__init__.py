"""Host runtime in C++ (``libmetrale_host.so``, built in-tree by ``native/build.py`` with g++):

* ``NativeBlockAllocator`` / ``NativeRadixTree``: the KV block allocator and the radix prefix
  index, drop-in for ``cache.block_pool.BlockAllocator`` / ``cache.radix.RadixTree`` (those
  Python classes stay as the behavioural oracle of the differential tests).
* ``NativeJsonGrammar``: byte-level JSON pushdown recogniser with a whole-vocabulary token mask
  fill (constrained decoding for ``response_format``).
* ``NativePda``: pushdown matcher for grammars compiled by the ``grammar`` package (EBNF, regex,
  JSON Schema, structural tags) with an exact, memoised whole-vocabulary mask and rollback.
* ``read_ranges``: multi-threaded ``pread`` (optionally O_DIRECT) of byte ranges of a file into
  caller-owned memory (pinned staging of the checkpoint loader).

``available()`` says whether the library is present; ``METRALE_NATIVE_RUNTIME=0`` keeps the
engine on the Python implementations. Role of the reference's Rust runtime crates
(``crates/cache``, ``crates/grammar``, ``crates/model-weights/src/fast_weights``).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.block_pool import NoFreeBlocks
from ..cache.radix import PrefixMatch

_HERE = Path(__file__).resolve().parent
_lib = None
_tried = False

_I32P = C.POINTER(C.c_int32)
_I64P = C.POINTER(C.c_int64)
_U8P = C.POINTER(C.c_uint8)


def _load():
    global _lib, _tried
    if _tried:
        return _lib
    _tried = True
    path = _HERE / "libmetrale_host.so"
    if not path.exists() and os.environ.get("METRALE_B200_AUTOBUILD", "1") != "0":
        try:
            from . import build as _b
            _b.build()
        except Exception:
            return None
    if not path.exists():
        return None
    L = C.CDLL(str(path))
    sig = {
        "mrt_alloc_create": (C.c_void_p, [C.c_int32]),
        "mrt_alloc_destroy": (None, [C.c_void_p]),
        "mrt_alloc_num_free": (C.c_int32, [C.c_void_p]),
        "mrt_alloc_refcount": (C.c_int32, [C.c_void_p, C.c_int32]),
        "mrt_alloc_take": (C.c_int32, [C.c_void_p, C.c_int32, _I32P]),
        "mrt_alloc_incref": (C.c_int32, [C.c_void_p, _I32P, C.c_int32]),
        "mrt_alloc_release": (C.c_int32, [C.c_void_p, _I32P, C.c_int32, _I32P]),
        "mrt_radix_create": (C.c_void_p, [C.c_void_p, C.c_int32, C.c_int32]),
        "mrt_radix_destroy": (None, [C.c_void_p]),
        "mrt_radix_match": (C.c_int32, [C.c_void_p, _I32P, C.c_int32, C.c_int64, C.c_int32, _I32P, _I64P]),
        "mrt_radix_insert": (C.c_int32, [C.c_void_p, _I32P, C.c_int32, _I32P, C.c_int32, C.c_int64, _I64P, _I64P, C.c_int32]),
        "mrt_radix_evict": (C.c_int32, [C.c_void_p, C.c_int32]),
        "mrt_radix_evictable": (C.c_int32, [C.c_void_p]),
        "mrt_radix_drain_evicted_snapshots": (C.c_int32, [C.c_void_p, _I64P, C.c_int32]),
        "mrt_radix_stats": (None, [C.c_void_p, _I64P]),
        "mrt_radix_clear": (None, [C.c_void_p]),
        "mrt_vocab_create": (C.c_void_p, [C.c_int32, _U8P, _I64P]),
        "mrt_vocab_destroy": (None, [C.c_void_p]),
        "mrt_json_create": (C.c_void_p, [C.c_int32]),
        "mrt_json_clone": (C.c_void_p, [C.c_void_p]),
        "mrt_json_destroy": (None, [C.c_void_p]),
        "mrt_json_complete": (C.c_int32, [C.c_void_p]),
        "mrt_json_feed": (C.c_int32, [C.c_void_p, _U8P, C.c_int32]),
        "mrt_json_fill_mask": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, _U8P, C.c_int32]),
        "mrt_json_advance": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32]),
        "mrt_pda_grammar_create": (C.c_void_p, [C.c_int32, _I32P, C.c_int32, _I32P, _I32P, _I32P, _I32P, _I32P,
                                                C.c_int32, _I32P, C.c_int32]),
        "mrt_pda_grammar_destroy": (None, [C.c_void_p]),
        "mrt_pda_create": (C.c_void_p, [C.c_void_p]),
        "mrt_pda_destroy": (None, [C.c_void_p]),
        "mrt_pda_reset": (None, [C.c_void_p]),
        "mrt_pda_complete": (C.c_int32, [C.c_void_p]),
        "mrt_pda_feed": (C.c_int32, [C.c_void_p, _U8P, C.c_int32]),
        "mrt_pda_advance": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32]),
        "mrt_pda_rollback": (C.c_int32, [C.c_void_p, C.c_int32]),
        "mrt_pda_stats": (None, [C.c_void_p, _I64P]),
        "mrt_pda_fill_mask": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, _U8P, C.c_int32]),
        "mrt_read_ranges": (C.c_int64, [C.c_char_p, C.c_int32, _I64P, _I64P, C.POINTER(C.c_void_p), C.c_int32, C.c_int32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _lib = L
    return _lib


def available() -> bool:
    return os.environ.get("METRALE_NATIVE_RUNTIME", "1") != "0" and _load() is not None


def _arr(xs: Sequence[int]):
    return (C.c_int32 * max(1, len(xs)))(*xs)


# ---------------------------------------------------------------------------- allocator
class _RefView:
    """``alloc.refcount[b]`` as the Python allocator exposes it (read-only)."""

    def __init__(self, owner):
        self._o = owner

    def __getitem__(self, b: int) -> int:
        return _lib.mrt_alloc_refcount(self._o._h, int(b))


class NativeBlockAllocator:
    def __init__(self, num_blocks: int):
        assert num_blocks >= 2
        L = _load()
        if L is None:
            raise RuntimeError("native host runtime is not built")
        self.num_blocks = num_blocks
        self._h = C.c_void_p(L.mrt_alloc_create(num_blocks))
        self.refcount = _RefView(self)

    def __del__(self):
        if _lib is not None and getattr(self, "_h", None):
            _lib.mrt_alloc_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return _lib.mrt_alloc_num_free(self._h)

    @property
    def num_used(self) -> int:
        return self.num_blocks - 1 - self.num_free

    def alloc(self, n: int = 1) -> List[int]:
        out = (C.c_int32 * max(1, n))()
        if _lib.mrt_alloc_take(self._h, n, out) < 0:
            raise NoFreeBlocks(f"need {n} blocks, {self.num_free} free")
        return list(out[:n])

    def incref(self, blocks) -> None:
        blocks = list(blocks)
        if blocks and _lib.mrt_alloc_incref(self._h, _arr(blocks), len(blocks)) < 0:
            raise AssertionError("incref on a free block")

    def free(self, blocks) -> List[int]:
        blocks = list(blocks)
        if not blocks:
            return []
        out = (C.c_int32 * len(blocks))()
        n = _lib.mrt_alloc_release(self._h, _arr(blocks), len(blocks), out)
        if n < 0:
            raise AssertionError("double free of a block")
        return list(out[:n])


# ---------------------------------------------------------------------------- radix index
class NativeRadixTree:
    def __init__(self, allocator: NativeBlockAllocator, block_size: int, needs_snapshot: bool = False,
                 on_snapshot_evict=None):
        assert isinstance(allocator, NativeBlockAllocator), "the native index shares the native allocator"
        self.alloc, self.block_size = allocator, block_size
        self.needs_snapshot, self.on_snapshot_evict = needs_snapshot, on_snapshot_evict
        self._h = C.c_void_p(_lib.mrt_radix_create(allocator._h, block_size, int(needs_snapshot)))
        self._adapters: Dict[Hashable, int] = {None: 0}

    def __del__(self):
        if _lib is not None and getattr(self, "_h", None):
            _lib.mrt_radix_destroy(self._h)
            self._h = None

    def _aid(self, adapter: Hashable) -> int:
        if adapter not in self._adapters:
            self._adapters[adapter] = len(self._adapters)
        return self._adapters[adapter]

    def match(self, tokens: Sequence[int], adapter: Hashable = None, max_tokens: Optional[int] = None) -> PrefixMatch:
        n = len(tokens)
        out = (C.c_int32 * max(1, n // self.block_size))()
        snap = C.c_int64(-1)
        k = _lib.mrt_radix_match(self._h, _arr(tokens), n, self._aid(adapter), -1 if max_tokens is None else max_tokens,
                                 out, C.byref(snap))
        return PrefixMatch(list(out[:k]), k * self.block_size, None if snap.value < 0 else int(snap.value))

    def insert(self, tokens: Sequence[int], blocks: Sequence[int], adapter: Hashable = None,
               snapshots: Optional[Dict[int, int]] = None) -> int:
        sp = list((snapshots or {}).items())
        pos = (C.c_int64 * max(1, len(sp)))(*[p for p, _ in sp])
        ids = (C.c_int64 * max(1, len(sp)))(*[i for _, i in sp])
        return _lib.mrt_radix_insert(self._h, _arr(tokens), len(tokens), _arr(blocks), len(blocks),
                                     self._aid(adapter), pos, ids, len(sp))

    def _drain(self) -> None:
        buf = (C.c_int64 * 64)()
        while True:
            n = _lib.mrt_radix_drain_evicted_snapshots(self._h, buf, 64)
            for i in range(n):
                if self.on_snapshot_evict:
                    self.on_snapshot_evict(int(buf[i]))
            if n < 64:
                break

    def evict(self, num_blocks: int) -> int:
        n = _lib.mrt_radix_evict(self._h, num_blocks)
        self._drain()
        return n

    def evictable_blocks(self) -> int:
        return _lib.mrt_radix_evictable(self._h)

    def clear(self) -> None:
        _lib.mrt_radix_clear(self._h)
        self._drain()

    def stats(self) -> dict:
        s = (C.c_int64 * 5)()
        _lib.mrt_radix_stats(self._h, s)
        return {"nodes": int(s[0]), "queries": int(s[1]), "hits": int(s[2]), "hit_tokens": int(s[3])}

    @property
    def num_nodes(self) -> int:
        return self.stats()["nodes"]


# ---------------------------------------------------------------------------- JSON grammar
class _Vocab:
    _cache: Dict[int, "_Vocab"] = {}

    def __init__(self, tokenizer, vocab_size: int):
        blobs, offs = [], [0]
        for t in range(vocab_size):
            try:
                b = tokenizer.token_bytes(t) or b""
            except Exception:
                b = b""
            blobs.append(b)
            offs.append(offs[-1] + len(b))
        blob = b"".join(blobs) or b"\0"
        self.n = vocab_size
        self._blob = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        self._offs = (C.c_int64 * len(offs))(*offs)
        self.h = C.c_void_p(_lib.mrt_vocab_create(vocab_size, self._blob, self._offs))

    @classmethod
    def of(cls, tokenizer, vocab_size: int) -> "_Vocab":
        key = (id(tokenizer), vocab_size)
        if key not in cls._cache:
            cls._cache[key] = cls(tokenizer, vocab_size)
        return cls._cache[key]


class NativeJsonGrammar:
    """Same interface as ``server.grammar.TokenGrammar`` (``allowed_mask`` / ``advance``), with an
    exact mask over the whole vocabulary instead of a probe of the highest logits."""

    def __init__(self, tokenizer, eos_token_id: Optional[int] = None, require_object: bool = True,
                 vocab_size: Optional[int] = None):
        if _load() is None:
            raise RuntimeError("native host runtime is not built")
        self.tk, self.eos, self.require_object = tokenizer, eos_token_id, require_object
        self.vocab = _Vocab.of(tokenizer, vocab_size or tokenizer.vocab_size)
        self._h = C.c_void_p(_lib.mrt_json_create(int(require_object)))
        self._history: List[int] = []

    def __del__(self):
        if _lib is not None and getattr(self, "_h", None):
            _lib.mrt_json_destroy(self._h)
            self._h = None

    # the matcher lives in native memory: a copy sent to another rank is rebuilt by replaying the
    # tokens accepted so far
    def __getstate__(self):
        return {"tk": self.tk, "eos": self.eos, "require_object": self.require_object, "n": self.vocab.n,
                "history": list(self._history)}

    def __setstate__(self, st):
        self.__init__(st["tk"], st["eos"], st["require_object"], st["n"])
        for t in st["history"]:
            self.advance(t)

    def observe_logits(self, row) -> None:      # interface parity; the exact fill needs no hint
        pass

    def allowed_mask(self, vocab: int) -> torch.Tensor:
        mask = torch.zeros(vocab, dtype=torch.uint8)
        ptr = C.cast(mask.data_ptr(), _U8P)
        n = _lib.mrt_json_fill_mask(self._h, self.vocab.h, -1 if self.eos is None else self.eos, ptr, vocab)
        if n == 0 and self.eos is not None and self.eos < vocab:
            mask[self.eos] = 1
        return mask.bool()

    def advance(self, tid: int) -> None:
        if tid != self.eos:
            _lib.mrt_json_advance(self._h, self.vocab.h, int(tid))
            self._history.append(int(tid))

    def rollback(self, n: int) -> None:
        """Forgets the last n accepted tokens (rebuilds the recogniser by replaying the rest)."""
        keep = self._history[:max(0, len(self._history) - n)]
        _lib.mrt_json_destroy(self._h)
        self._h = C.c_void_p(_lib.mrt_json_create(int(self.require_object)))
        self._history = []
        for t in keep:
            self.advance(t)

    def is_complete(self) -> bool:
        return bool(_lib.mrt_json_complete(self._h))

    def feed_bytes(self, bs: bytes) -> bool:
        buf = (C.c_uint8 * max(1, len(bs))).from_buffer_copy(bs or b"\0")
        return _lib.mrt_json_feed(self._h, buf, len(bs)) == len(bs)


# ---------------------------------------------------------------------------- pushdown grammar
def has_pda() -> bool:
    return _load() is not None and hasattr(_lib, "mrt_pda_create")


class _NativeGrammar:
    """The compiled tables of a ``grammar.CompiledGrammar`` in native memory (shared by matchers)."""

    def __init__(self, g):
        def arr(xs):
            return (C.c_int32 * max(1, len(xs)))(*xs)
        self.h = C.c_void_p(_lib.mrt_pda_grammar_create(
            g.n_nodes, arr(g.edge_begin), len(g.edge_kind), arr(g.edge_kind), arr(g.edge_a), arr(g.edge_b),
            arr(g.edge_to), arr(g.final), len(g.rule_start), arr(g.rule_start), g.root))
        if not self.h:
            raise ValueError("malformed compiled grammar")

    def __del__(self):
        if _lib is not None and getattr(self, "h", None):
            _lib.mrt_pda_grammar_destroy(self.h)
            self.h = None


class NativePda:
    """Pushdown matcher over a compiled grammar with an exact whole-vocabulary mask and rollback
    (``grammar.TokenMatcher`` wraps it)."""

    def __init__(self, grammar, tokenizer=None, vocab_size: Optional[int] = None):
        if not has_pda():
            raise RuntimeError("native host runtime is not built")
        if grammar._native is None:
            grammar._native = _NativeGrammar(grammar)
        self._g = grammar._native                     # keeps the tables alive
        self.vocab = _Vocab.of(tokenizer, vocab_size or tokenizer.vocab_size) if tokenizer is not None else None
        self._h = C.c_void_p(_lib.mrt_pda_create(self._g.h))

    def __del__(self):
        if _lib is not None and getattr(self, "_h", None):
            _lib.mrt_pda_destroy(self._h)
            self._h = None

    def fill_mask(self, vocab: int, eos: Optional[int]) -> torch.Tensor:
        mask = torch.zeros(vocab, dtype=torch.uint8)
        _lib.mrt_pda_fill_mask(self._h, self.vocab.h, -1 if eos is None else eos,
                               C.cast(mask.data_ptr(), _U8P), vocab)
        return mask.bool()

    def advance(self, tid: int) -> bool:
        return bool(_lib.mrt_pda_advance(self._h, self.vocab.h, int(tid)))

    def rollback(self, n: int) -> int:
        return int(_lib.mrt_pda_rollback(self._h, int(n)))

    def is_complete(self) -> bool:
        return bool(_lib.mrt_pda_complete(self._h))

    def feed(self, bs: bytes) -> bool:
        buf = (C.c_uint8 * max(1, len(bs))).from_buffer_copy(bs or b"\0")
        return bool(_lib.mrt_pda_feed(self._h, buf, len(bs)))

    def reset(self) -> None:
        _lib.mrt_pda_reset(self._h)

    def stats(self) -> Dict[str, int]:
        out = (C.c_int64 * 4)()
        _lib.mrt_pda_stats(self._h, out)
        return {"items": out[0], "frames": out[1], "mask_cache_hits": out[2], "mask_cache_misses": out[3]}


# ---------------------------------------------------------------------------- file reader
def read_ranges(path: str, offsets: Sequence[int], sizes: Sequence[int], dst_ptrs: Sequence[int],
                threads: int = 8, direct: bool = False) -> int:
    """Reads ``sizes[i]`` bytes at ``offsets[i]`` of ``path`` into the memory at ``dst_ptrs[i]``."""
    L = _load()
    if L is None:
        raise RuntimeError("native host runtime is not built")
    n = len(offsets)
    off = (C.c_int64 * max(1, n))(*offsets)
    sz = (C.c_int64 * max(1, n))(*sizes)
    dst = (C.c_void_p * max(1, n))(*dst_ptrs)
    r = L.mrt_read_ranges(os.fsencode(path), n, off, sz, dst, threads, int(direct))
    if r < 0:
        raise OSError(-r, os.strerror(-r), path)
    return int(r)
