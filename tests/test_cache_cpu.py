"""Block allocator, radix prefix cache and recurrent-state pool (CPU). Mirrors the reference's
cache tests (``crates/kv-cache`` / ``crates/prefix-cache`` unit tests: refcounts, LRU leaf
eviction, adapter isolation, snapshot-gated matches)."""
import pytest
import torch

from metrale_inference_alpha_b200.cache.block_pool import (BlockAllocator, KvCacheConfig, NoFreeBlocks,
                                                             PagedKvCache)
from metrale_inference_alpha_b200.cache.radix import RadixTree
from metrale_inference_alpha_b200.cache.state_pool import StatePool


def test_allocator_refcounts_and_null_block():
    a = BlockAllocator(8)
    assert a.num_free == 7
    b = a.alloc(3)
    assert 0 not in b and a.num_used == 3
    a.incref(b[:1])
    assert a.free(b) == b[1:]
    assert a.num_used == 1
    assert a.free(b[:1]) == b[:1] and a.num_used == 0
    assert a.free([0]) == []                      # the null block is never released
    with pytest.raises(NoFreeBlocks):
        a.alloc(8)
    with pytest.raises(AssertionError):
        a.free(b[:1])                             # double free is caught


def test_radix_match_insert_and_never_the_whole_prompt():
    a = BlockAllocator(32)
    t = RadixTree(a, 4)
    toks = list(range(1, 17))                     # 4 full blocks
    blocks = a.alloc(4)
    assert t.insert(toks, blocks) == 4
    m = t.match(toks)
    assert m.tokens == 12 and m.blocks == blocks[:3]    # one token must remain to prefill
    m2 = t.match(toks + [99])
    assert m2.tokens == 16
    m3 = t.match([1, 2, 3, 4, 9, 9, 9, 9, 9])
    assert m3.tokens == 4
    assert t.match([7, 7, 7, 7, 7]).tokens == 0
    # second insert of the same chunks adopts nothing
    dup = a.alloc(4)
    assert t.insert(toks, dup) == 0
    st = t.stats()
    assert st["queries"] == 4 and st["hits"] == 3


def test_radix_adapter_isolation():
    a = BlockAllocator(32)
    t = RadixTree(a, 4)
    toks = list(range(1, 10))
    t.insert(toks, a.alloc(2), adapter="lora-a")
    assert t.match(toks, adapter="lora-a").tokens == 8
    assert t.match(toks, adapter="lora-b").tokens == 0
    assert t.match(toks).tokens == 0


def test_radix_lru_eviction_frees_only_unreferenced_leaves():
    a = BlockAllocator(16)
    t = RadixTree(a, 4)
    s1, s2 = list(range(1, 9)), list(range(101, 109))
    b1, b2 = a.alloc(2), a.alloc(2)
    t.insert(s1, b1)
    t.insert(s2, b2)
    a.free(b1)
    a.free(b2)                                    # only the tree holds them now
    held = t.match(s2 + [0])                      # a live sequence references s2's blocks; s2 is also most recent
    free0 = a.num_free
    assert t.evict(4) == 2                        # only s1's two blocks can go
    assert a.num_free == free0 + 2
    assert t.match(s1 + [0]).tokens == 0
    a.free(held.blocks)
    assert t.evict(4) == 2
    assert a.num_used == 0


def test_radix_snapshot_gated_match():
    a = BlockAllocator(16)
    t = RadixTree(a, 4, needs_snapshot=True)
    toks = list(range(1, 14))
    t.insert(toks, a.alloc(3), snapshots={8: 5})
    m = t.match(toks)
    assert m.tokens == 8 and m.snapshot == 5  # deepest node that has recurrent state
    t2 = RadixTree(a, 4, needs_snapshot=True)
    t2.insert(toks, a.alloc(3))
    assert t2.match(toks).tokens == 0


def test_paged_kv_layout_copy_and_gather():
    cfg = KvCacheConfig(num_layers=2, kv_heads=2, head_dim=8, block_size=4, dtype="bf16")
    kv = PagedKvCache(cfg, 6, "cpu")
    assert kv.bytes() == 6 * cfg.block_bytes()
    kv.k[0][1].fill_(3.0)
    kv.copy_block(1, 2)
    assert torch.equal(kv.k[0][2], kv.k[0][1])
    data = kv.gather_blocks([1, 2])
    kv.k[0][1].zero_()
    kv.scatter_blocks([1, 2], data)
    assert float(kv.k[0][1].float().mean()) == 3.0


def test_state_pool_slots_snapshots_and_export():
    p = StatePool([((4, 3), (2, 5, 6))], num_slots=4, num_snapshots=2)
    s = p.alloc()
    assert s != 0 and p.num_free == 2
    p.conv[0][s].fill_(1.5)
    p.ssm[0][s].fill_(-2.0)
    sid = p.snapshot(s)
    p.reset(s)
    assert float(p.conv[0][s].abs().sum()) == 0.0
    p.restore(sid, s)
    assert float(p.conv[0][s].mean()) == 1.5 and float(p.ssm[0][s].mean()) == -2.0
    blob = p.export_slot(s)
    s2 = p.alloc()
    p.import_slot(s2, blob)
    assert torch.equal(p.ssm[0][s2], p.ssm[0][s])
    p.release_snapshot(sid)
    assert p.snapshot(s) is not None and p.snapshot(s) is not None and p.snapshot(s) is None   # pool of two
    p.free(s)
    p.free(s2)
    assert p.num_free == 3
