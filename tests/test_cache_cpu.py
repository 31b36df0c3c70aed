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


# ---------------------------------------------------------------- FP8 KV scales
def test_kv_scale_keys_resolve_three_spellings_and_refuse_ambiguity():
    from metrale_inference_alpha_b200.weights.kv_scales import kv_scale_census, load_kv_scales, resolve_kv_scale_keys
    from metrale_inference_alpha_b200.weights.source import DictSource
    import torch
    p = "model.layers.3.self_attn"
    for spelling, ks, vs in (("k_proj_output", "k_proj.k_scale", "v_proj.v_scale"), ("attn_module", "attn.k_scale", "attn.v_scale"),
                             ("bare", "k_scale", "v_scale")):
        src = DictSource({f"{p}.{ks}": torch.tensor(0.02), f"{p}.{vs}": torch.tensor([0.5])})
        assert resolve_kv_scale_keys(src.has, p) == (spelling, f"{p}.{ks}", f"{p}.{vs}")
        got = load_kv_scales(src, {3: p, 4: "model.layers.4.self_attn"})
        assert set(got) == {3} and abs(got[3][0] - 0.02) < 1e-7 and got[3][1] == 0.5
        assert kv_scale_census(src, {3: p, 4: "model.layers.4.self_attn"}) == {spelling: 1, "none": 1}
    with pytest.raises(ValueError, match="but not"):
        resolve_kv_scale_keys(DictSource({f"{p}.k_scale": torch.tensor(1.0)}).has, p)
    two = DictSource({f"{p}.k_scale": torch.tensor(1.0), f"{p}.v_scale": torch.tensor(1.0),
                      f"{p}.attn.k_scale": torch.tensor(1.0), f"{p}.attn.v_scale": torch.tensor(1.0)})
    with pytest.raises(ValueError, match="2 ways"):
        resolve_kv_scale_keys(two.has, p)
    with pytest.raises(ValueError, match="non-positive"):
        load_kv_scales(DictSource({f"{p}.k_scale": torch.tensor(0.0), f"{p}.v_scale": torch.tensor(1.0)}), {3: p})


def test_engine_takes_fp8_kv_scales_from_the_checkpoint():
    import torch
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.weights.source import DictSource, SyntheticSource
    cfg = preset("tiny-dense", kv_dtype="fp8")
    syn = SyntheticSource(cfg, seed=0)
    t = {n: syn.get(n) for n in syn.names()}
    t["model.layers.0.self_attn.k_proj.k_scale"] = torch.tensor(0.03)
    t["model.layers.0.self_attn.v_proj.v_scale"] = torch.tensor(0.01)
    eng = LLMEngine(EngineArgs(model=cfg, device="cpu", max_model_len=128, num_kv_blocks=32), source=DictSource(t))
    kv = eng.runner.kv
    assert eng.runner.kv_scales_loaded == 1
    assert abs(float(kv.k_scale[0]) - 0.03) < 1e-7 and abs(float(kv.v_scale[0]) - 0.01) < 1e-7
    assert float(kv.k_scale[1]) == 1.0
    out = eng.generate([[5, 6, 7, 8, 9]], SamplingParams(max_tokens=4))[0]
    assert len(out.output_ids) == 4


def test_online_fp8_kv_calibration_freezes_rescales_and_holds_graphs_back():
    """Scales start provisional, the window's entries are re-encoded at the frozen scale
    amax * headroom / 448, and CUDA graphs are reported not ready until then."""
    import torch
    from metrale_inference_alpha_b200.cache.fp8_calibration import PROVISIONAL_SCALE
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.ops import reference as ref
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    cfg = preset("tiny-dense", kv_dtype="fp8")
    prompt = [(5 * j) % 200 + 1 for j in range(40)]
    eng = LLMEngine(EngineArgs(model=cfg, device="cpu", max_model_len=128, num_kv_blocks=32, fp8_kv_calibration_tokens=48,
                               fp8_kv_headroom=1.25, enable_prefix_caching=False))
    r = eng.runner
    assert r.kv_cal is not None and not r.kv_cal.frozen and float(r.kv.k_scale[0]) == PROVISIONAL_SCALE
    def ready():                                           # a CPU engine never uses graphs: only the readiness rule is checked
        r.use_graphs = True
        try:
            return r.graphs_ready()
        finally:
            r.use_graphs = False
    assert not ready()
    eng.add_request(prompt, SamplingParams(max_tokens=20))
    eng.step()                                             # prefill: 40 tokens observed, window not reached
    cal = r.kv_cal
    assert cal is not None and cal.observed == 40
    amax_k = float(cal.amax[0][0])
    assert amax_k > 0
    while eng.has_work():
        eng.step()
    assert r.kv_cal is None and cal.frozen and ready()
    for i in range(cfg.num_layers):
        ks, vs = float(r.kv.k_scale[i]), float(r.kv.v_scale[i])
        assert abs(ks - float(cal.amax[i][0]) * 1.25 / 448) < 1e-9 and abs(vs - float(cal.amax[i][1]) * 1.25 / 448) < 1e-9
        assert ks not in (1.0, PROVISIONAL_SCALE)
    # the window's cached keys decode to the same values (to e4m3 rounding) as a cache written at the frozen scale from the start
    eng2 = LLMEngine(EngineArgs(model=cfg, device="cpu", max_model_len=128, num_kv_blocks=32, enable_prefix_caching=False))
    for i in range(cfg.num_layers):
        eng2.runner.kv.k_scale[i].copy_(r.kv.k_scale[i])
        eng2.runner.kv.v_scale[i].copy_(r.kv.v_scale[i])
    eng2.add_request(prompt, SamplingParams(max_tokens=1))
    eng2.step()
    a = ref.from_e4m3(r.kv.k[0][1:3]) * float(r.kv.k_scale[0])          # blocks 1, 2: positions 0..31 of the first sequence
    b = ref.from_e4m3(eng2.runner.kv.k[0][1:3]) * float(r.kv.k_scale[0])
    assert (a - b).abs().max().item() <= 0.13 * b.abs().max().item()


def test_state_snapshots_overflow_into_host_and_file_tiers(tmp_path):
    """Resident snapshot area of 2: further snapshots demote the least recently used resident one
    to host memory, and the host tier (budget of one slot) demotes its oldest to a file; every
    handle restores the exact state it captured, from whichever tier, and release cleans up."""
    import os
    import torch
    from metrale_inference_alpha_b200.cache.state_pool import StatePool
    pool = StatePool([((6, 3), (2, 4, 5))], num_slots=3, num_snapshots=2)
    pool.configure_tiers(host_tier_bytes=pool.bytes_per_slot(), tier_dir=str(tmp_path))
    handles, want = [], []
    for n in range(5):
        pool.conv[0][1].fill_(float(n))
        pool.ssm[0][1].fill_(float(10 + n))
        handles.append(pool.snapshot(1))
        want.append((float(n), float(10 + n)))
    assert None not in handles and len(set(handles)) == 5
    tiers = [pool._where[h][0] for h in handles]
    assert tiers.count("dev") == 2 and tiers.count("host") == 1 and tiers.count("file") == 2
    assert len(os.listdir(tmp_path)) == 2
    for h, (c, s) in zip(handles, want):
        pool.restore(h, 2)
        assert float(pool.conv[0][2].mean()) == c and float(pool.ssm[0][2].mean()) == s
    assert pool.tier_stats["restored_file"] == 2 and pool.tier_stats["restored_host"] == 1
    for h in handles:
        pool.release_snapshot(h)
    assert os.listdir(tmp_path) == [] and len(pool._snap_free) == 2 and pool._host_bytes == 0
    # without tiers a full area refuses, as before
    plain = StatePool([((6, 3), (2, 4, 5))], num_slots=3, num_snapshots=1)
    assert plain.snapshot(1) is not None and plain.snapshot(1) is None


def test_decode_ring_keeps_the_newest_entries_and_needs_an_exact_position():
    from metrale_inference_alpha_b200.scheduler.decode_ring import StateDecodeRing
    r = StateDecodeRing(3)
    dropped = [r.record(p, 100 + p) for p in (4, 8, 12, 16)]
    assert dropped == [None, None, None, 104] and r.positions() == [8, 12, 16]
    assert r.find(12).snapshot == 112 and r.find(10) is None
    assert r.last_at_or_before(15).token_position == 12
    assert r.record(12, 999) == 112                       # a re-generated position replaces its entry
    assert r.truncate_after(8) == [999, 116] and r.positions() == [8]
    assert StateDecodeRing(0).record(4, 7) == 7            # a disabled ring hands the snapshot straight back
