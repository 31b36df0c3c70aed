"""Storage tiers: KV blocks in files attended tile by tile, the low-rank block predictor, the byte
stores under them, expert paging and the file-backed row cache. CPU tensors take the fp32 restatement
of every kernel, so these tests cover the host logic; the kernels are compared with the same
restatements in the GPU tests."""
import math
import os

import pytest
import torch

from metrale_inference_alpha_b200.storage import kernels as SK
from metrale_inference_alpha_b200.storage.backend import (CascadeBackend, CommitLedger, FileBackend, KvLayout,
                                                           MemoryBackend, pinned_bytes)
from metrale_inference_alpha_b200.storage.high_speed_swap import (DiskBlocks, EvictionPolicy, HighSpeedSwap,
                                                                   HighSpeedSwapConfig, ModelDims, ResidentTail)


def _attention(q, k, v, scale):
    """q [Hq, D], k / v [n, Hkv, D] -> [Hq, D] fp32."""
    Hq, Hkv = q.shape[0], k.shape[1]
    G = Hq // Hkv
    out = torch.zeros(Hq, q.shape[1])
    for h in range(Hq):
        s = (k[:, h // G].float() @ q[h].float()) * scale
        out[h] = torch.softmax(s, 0) @ v[:, h // G].float()
    return out


def test_layout_offsets_are_dense_and_ordered():
    L = KvLayout(num_layers=2, num_blocks=3, block_size=4, kv_heads=2, head_dim=128, elem_bytes=2, fs_block=4096)
    assert L.group_payload == 4 * 128 * 2 and L.group_stride == 4096
    assert L.block_bytes == 2 * 2 * 4096 and L.bytes_per_layer == 3 * L.block_bytes
    offs = [L.file_offset(b, kind, h) for b in range(3) for kind in (0, 1) for h in range(2)]
    assert offs == sorted(offs) and len(set(offs)) == len(offs)
    ids = [L.group_id(layer, b, kind, h) for layer in range(2) for b in range(3) for kind in (0, 1) for h in range(2)]
    assert ids == list(range(2 * 3 * 2 * 2))
    with pytest.raises(IndexError):
        L.file_offset(3)


def test_file_backend_round_trip_and_cascade(tmp_path):
    L = KvLayout(1, 8, 4, 2, 128)
    fb = FileBackend(str(tmp_path / "kv"), L)
    bufs = []
    for b in range(6):
        buf = pinned_bytes(L.block_bytes)
        buf.copy_(torch.randint(0, 255, (L.block_bytes,), dtype=torch.uint8))
        bufs.append(buf.clone())
        fb.write_block(0, b, buf)
    out = [pinned_bytes(L.block_bytes) for _ in range(6)]
    for f in fb.read_blocks_async(0, list(range(6)), out):
        f.result()
    assert all(torch.equal(a, b) for a, b in zip(out, bufs))
    assert os.path.getsize(L.layer_path(str(tmp_path / "kv"), 0)) >= L.bytes_per_layer
    fb.close()
    # reopen without create: the data is still there
    fb = FileBackend(str(tmp_path / "kv"), L, create=False)
    one = pinned_bytes(L.block_bytes)
    fb.read_block(0, 3, one)
    assert torch.equal(one, bufs[3])
    # write-back tier of 2 slots in front of it
    cas = CascadeBackend(fb, slots=2)
    new = [torch.full((L.block_bytes,), 10 + i, dtype=torch.uint8) for i in range(3)]
    for i in range(3):
        cas.write_block(0, i, new[i])
    assert cas.stats["writebacks"] == 1                      # block 0 was written down when the tier filled
    cas.read_block(0, 2, one)
    assert torch.equal(one, new[2]) and cas.stats["hits"] == 1
    cas.read_block(0, 0, one)                                # a miss served by the files
    assert torch.equal(one, new[0]) and cas.stats["misses"] == 1
    cas.read_block(0, 5, one)
    assert torch.equal(one, bufs[5])
    cas.flush()
    fb.read_block(0, 1, one)
    assert torch.equal(one, new[1])
    cas.close()


def test_commit_ledger_cap():
    led = CommitLedger(100)
    a = led.reserve(60)
    assert a is not None and led.reserve(50) is None
    b = led.reserve(40)
    assert b is not None and led.committed == 100
    a.release()
    a.release()
    assert led.committed == 40 and led.reserve(60) is not None


def test_disk_block_ids_reuse_and_refcounts():
    d = DiskBlocks(3)
    a, b, c = d.alloc(), d.alloc(), d.alloc()
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(MemoryError):
        d.alloc()
    d.retain(b)
    assert d.release(b) is False and d.release(b) is True
    assert d.alloc() == b                                     # the free list comes before fresh ids
    with pytest.raises(KeyError):
        d.release(99)


def test_eviction_order_is_score_then_recency():
    ev = EvictionPolicy()
    for i, (score, epoch) in enumerate([(0.5, 1), (0.1, 3), (0.1, 2), (0.9, 0)]):
        ev.epoch = epoch
        ev.touch((0, i))
        ev.record_score((0, i), score)
    assert ev.rank([(0, i) for i in range(4)]) == [(0, 2), (0, 1), (0, 0), (0, 3)]


def test_tile_kernel_restatement_matches_softmax_attention():
    torch.manual_seed(0)
    Hq, Hkv, D, bs, nblk = 4, 2, 128, 4, 5
    pool_k = torch.randn(8, bs, Hkv, D).to(torch.bfloat16)
    pool_v = torch.randn(8, bs, Hkv, D).to(torch.bfloat16)
    q = torch.randn(2, Hq, D).to(torch.bfloat16)
    table = torch.tensor([[3, 1, 4, 0, 6], [2, 5, 7, 0, 0]], dtype=torch.int32)
    counts = torch.tensor([5, 3], dtype=torch.int32)
    last = torch.tensor([2, 4], dtype=torch.int32)
    state = SK.attn_state(2, Hq, D, "cpu")
    strides = SK.paged_strides(bs, Hkv, D)
    # two tiles: blocks 0..2 then 3..4 (sequence 1 has nothing in the second tile)
    SK.kv_tile_attn(q, pool_k, pool_v, table[:, :3].contiguous(), torch.tensor([3, 3], dtype=torch.int32), state,
                    Hkv=Hkv, block_size=bs, strides=strides,
                    last_valid=torch.tensor([bs, 4], dtype=torch.int32))
    SK.kv_tile_attn(q, pool_k, pool_v, table[:, 3:].contiguous(), torch.tensor([2, 0], dtype=torch.int32), state,
                    Hkv=Hkv, block_size=bs, strides=strides, last_valid=last)
    out = SK.attn_finalize(state[1], state[2]).float()
    for s, n in ((0, 4 * bs + 2), (1, 3 * bs)):
        ids = table[s, :counts[s]].long()
        k = pool_k[ids].reshape(-1, Hkv, D)[:n]
        v = pool_v[ids].reshape(-1, Hkv, D)[:n]
        ref = _attention(q[s], k, v, 1 / math.sqrt(D))
        assert torch.allclose(out[s], ref, atol=2e-2, rtol=2e-2)
    # a sequence that attended nothing finalises to zeros
    st = SK.attn_state(1, Hq, D, "cpu")
    assert torch.count_nonzero(SK.attn_finalize(st[1], st[2])) == 0


@pytest.mark.parametrize("kv_dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("use_files", [False, True])
def test_streamed_attention_equals_attention_over_the_whole_sequence(tmp_path, kv_dtype, use_files):
    torch.manual_seed(1)
    md = ModelDims(num_layers=2, num_q_heads=4, num_kv_heads=2, head_dim=128, kv_dtype=kv_dtype)
    cfg = HighSpeedSwapConfig(dir=str(tmp_path / "hss") if use_files else None, block_size=4, max_blocks_per_layer=32,
                              resident_blocks=9, tile_capacity=3, rank=16, host_cache_blocks=2 if use_files else 0,
                              max_seqs=2)
    hss = HighSpeedSwap(cfg, md)
    bs, Hkv, D = 4, 2, 128
    lens = [37, 18]                                          # tokens per sequence
    ks, vs = (0.5, 0.25) if kv_dtype != torch.bfloat16 else (1.0, 1.0)
    for layer in range(2):
        hss.set_kv_scales(layer, ks, vs)
    seqs = []
    for n in lens:
        k = (torch.randn(2, n, Hkv, D) * 0.5)
        v = torch.randn(2, n, Hkv, D)
        seqs.append((k.to(kv_dtype), v.to(kv_dtype)))
    q = torch.randn(2, len(lens), md.num_q_heads, D).to(torch.bfloat16)
    # offload every full block except the last two of each sequence, which stay in a paged pool
    pool_k = torch.zeros(2, 8, bs, Hkv, D, dtype=kv_dtype)
    pool_v = torch.zeros_like(pool_k)
    disk_ids, tails = [], []
    nxt = 0
    for s, n in enumerate(lens):
        nblk = (n + bs - 1) // bs
        cold = max(0, nblk - 2)
        ids = [hss.alloc_disk_block() for _ in range(cold)]
        for layer in range(2):
            k, v = seqs[s][0][layer], seqs[s][1][layer]
            for j, d in enumerate(ids):
                hss.offload_block(layer, d, k[j * bs:(j + 1) * bs], v[j * bs:(j + 1) * bs])
        tail_blocks = []
        for j in range(cold, nblk):
            m = min(bs, n - j * bs)
            for layer in range(2):
                pool_k[layer, nxt, :m] = seqs[s][0][layer][j * bs:j * bs + m]
                pool_v[layer, nxt, :m] = seqs[s][1][layer][j * bs:j * bs + m]
            tail_blocks.append(nxt)
            nxt += 1
        disk_ids.append(ids)
        tails.append(tail_blocks)
    table = torch.zeros(len(lens), 2, dtype=torch.int32)
    for s, t in enumerate(tails):
        table[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
    counts = torch.tensor([len(t) for t in tails], dtype=torch.int32)
    last = torch.tensor([n - ((n + bs - 1) // bs - 1) * bs for n in lens], dtype=torch.int32)
    raw = (lambda t: t.view(torch.uint8)) if kv_dtype != torch.bfloat16 else (lambda t: t)
    for step in range(2):                                     # the second step hits resident slots
        for layer in range(2):
            tail = ResidentTail(raw(pool_k[layer]), raw(pool_v[layer]), table, counts, last, SK.paged_strides(bs, Hkv, D))
            out = hss.attend_layer(layer, q[layer], disk_ids, tail=tail).float()
            for s, n in enumerate(lens):
                k = seqs[s][0][layer].float() * ks
                v = seqs[s][1][layer].float() * vs
                ref = _attention(q[layer, s], k, v, 1 / math.sqrt(D))
                assert torch.allclose(out[s], ref, atol=3e-2, rtol=3e-2), (layer, s, (out[s] - ref).abs().max())
    assert hss.stats["evictions"] > 0 and hss.stats["slot_hits"] > 0 and hss.stats["tiles"] >= 8
    # the predictor recorded a score for every offloaded block of the last layer
    assert all((1, d) in hss.eviction.score for ids in disk_ids for d in ids)
    # releasing a block frees its id and its slots
    first = disk_ids[0][0]
    hss.release_disk_block(first)
    assert hss.pool.slot_of((0, first)) is None and hss.alloc_disk_block() == first
    hss.close()


def test_predictor_ranks_the_block_that_holds_the_matching_key():
    torch.manual_seed(2)
    md = ModelDims(1, 4, 2, 128)
    cfg = HighSpeedSwapConfig(block_size=4, max_blocks_per_layer=16, resident_blocks=4, tile_capacity=2, rank=32, max_seqs=1)
    hss = HighSpeedSwap(cfg, md)
    q = torch.randn(1, 4, 128)
    ids = []
    for j in range(6):
        k = torch.randn(4, 2, 128) * 0.1
        if j == 4:
            k[2, 1] = q[0, 3] * 2.0                         # head 3 belongs to kv head 1
        d = hss.alloc_disk_block()
        hss.offload_block(0, d, k.to(torch.bfloat16), torch.randn(4, 2, 128).to(torch.bfloat16))
        ids.append(d)
    hss.attend_layer(0, q.to(torch.bfloat16), [ids])
    scores = [hss.eviction.score[(0, d)] for d in ids]
    assert max(range(6), key=lambda j: scores[j]) == 4
    # with the pool full, the victim is never the important block
    order = hss.eviction.rank([k for k in hss.pool.lookup])
    assert order[-1] == (0, ids[4]) or (0, ids[4]) not in hss.pool.lookup


def test_thread_local_installation():
    md = ModelDims(1, 2, 2, 128)
    hss = HighSpeedSwap(HighSpeedSwapConfig(block_size=4, max_blocks_per_layer=4, resident_blocks=2, tile_capacity=1,
                                            max_seqs=1), md)
    assert HighSpeedSwap.with_local(lambda h: h) is None
    hss.install_local()
    assert HighSpeedSwap.with_local(lambda h: h.cfg.block_size) == 4
    HighSpeedSwap.uninstall_local()
    assert HighSpeedSwap.with_local(lambda h: h) is None


def test_config_range_checks():
    with pytest.raises(ValueError):
        HighSpeedSwapConfig(rank=128).validate(ModelDims(1, 4, 2, 128))
    with pytest.raises(ValueError):
        HighSpeedSwapConfig().validate(ModelDims(1, 4, 2, 96))
    with pytest.raises(ValueError):
        HighSpeedSwapConfig(tile_capacity=100, resident_blocks=10).validate(ModelDims(1, 4, 2, 128))
    with pytest.raises(ValueError):
        HighSpeedSwapConfig().validate(ModelDims(1, 5, 2, 128))


# ----------------------------------------------------------------------------- expert store / paging
def _ffn(seed, fmt="fp8_row", H=64, I=128):
    from metrale_inference_alpha_b200 import ops
    from metrale_inference_alpha_b200.weights.loader import FfnW
    g = torch.Generator().manual_seed(seed)
    gu = ops.make_weight(torch.randn(2 * I, H, generator=g) * 0.1, fmt)
    dn = ops.make_weight(torch.randn(H, I, generator=g) * 0.1, fmt)
    return FfnW(gu, dn, False, 0.0)


@pytest.mark.parametrize("fmt", ["bf16", "fp8_row", "nvfp4"])
def test_expert_records_round_trip(tmp_path, fmt):
    from metrale_inference_alpha_b200.storage import expert_store as XS
    layers = [[_ffn(10 * l + e, fmt) for e in range(3)] for l in range(2)]
    spec = XS.write_store(str(tmp_path / "x"), layers)
    spec.check()
    assert spec.record_stride % 4096 == 0 and all(s.offset % 256 == 0 for s in spec.subs)
    rd = XS.ExpertFileReader(str(tmp_path / "x"))
    assert (rd.num_layers, rd.num_experts) == (2, 3)
    buf = torch.empty(spec.record_stride, dtype=torch.uint8)
    rd.read_record(1, 2, buf)
    views, scal = XS.unpack_record(rd.spec, buf, 1, 2)
    assert torch.equal(views["gate_up.data"], layers[1][2].gate_up.data)
    if fmt != "bf16":
        assert torch.equal(views["down.scale"].view(torch.uint8), layers[1][2].down.scale.view(torch.uint8))
    assert scal["gate_up.gscale"] == pytest.approx(layers[1][2].gate_up.gscale)
    with pytest.raises(ValueError):
        XS.unpack_record(rd.spec, buf, 1, 1)                  # the header names another expert
    with pytest.raises(IndexError):
        rd.read_record(2, 0, buf)
    rd.close()
    # a manifest of another version is refused
    import json
    m = json.load(open(tmp_path / "x" / "manifest.json"))
    m["version"] = 99
    json.dump(m, open(tmp_path / "x" / "manifest.json", "w"))
    with pytest.raises(ValueError):
        XS.ExpertFileReader(str(tmp_path / "x"))


def test_paged_arena_clock_eviction_and_waves(tmp_path):
    from metrale_inference_alpha_b200.storage import expert_store as XS
    layers = [[_ffn(e) for e in range(6)]]
    XS.write_store(str(tmp_path / "x"), layers)
    pg = XS.PagedExperts(XS.ExpertFileReader(str(tmp_path / "x")), slots=3)
    idx = torch.tensor([[0, 1], [1, 2]], dtype=torch.int32)
    (w0,) = list(pg.waves(0, idx))
    assert pg.stats["loads"] == 3 and sorted(w0.flatten().tolist()) == sorted([pg.lookup[(0, e)] for e in (0, 1, 1, 2)])
    for e in (0, 1, 2):
        f = pg.slot_ffn(pg.lookup[(0, e)])
        assert torch.equal(f.gate_up.data, layers[0][e].gate_up.data) and torch.equal(f.down.scale, layers[0][e].down.scale)
    (w1,) = list(pg.waves(0, torch.tensor([[1, 4]], dtype=torch.int32)))          # one hit, one load + eviction
    assert pg.stats["hits"] == 1 and pg.stats["evictions"] == 1 and (0, 1) in pg.lookup and (0, 4) in pg.lookup
    # five distinct experts through three slots: two waves, every id appears in exactly one of them
    idx = torch.tensor([[0, 1, 2, 3, 5]], dtype=torch.int32)
    ws = list(pg.waves(0, idx))
    assert len(ws) == 2
    covered = torch.stack([(w >= 0) for w in ws]).sum(0)
    assert torch.equal(covered, torch.ones_like(covered))


def test_engine_with_paged_experts_matches_resident_experts(tmp_path):
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    prompts = [list(range(5, 25)), list(range(40, 52))]
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    base = LLMEngine(EngineArgs(model="tiny-hybrid-moe", device="cpu", num_kv_blocks=64, max_num_seqs=4))
    want = [o.output_ids for o in base.generate(prompts, sp)]
    eng = LLMEngine(EngineArgs(model="tiny-hybrid-moe", device="cpu", num_kv_blocks=64, max_num_seqs=4,
                               expert_arena_slots=3, expert_store_dir=str(tmp_path / "experts")))
    got = [o.output_ids for o in eng.generate(prompts, sp)]
    assert got == want
    st = eng.paged_experts.stats
    assert st["loads"] > 3 and st["evictions"] > 0 and st["waves"] > 0
    assert os.path.exists(tmp_path / "experts" / "manifest.json")


# ----------------------------------------------------------------------------- row cache
def test_row_cache_faults_pins_and_evicts(tmp_path):
    from metrale_inference_alpha_b200.storage.row_cache import RowCache
    table = torch.randn(50, 24).to(torch.bfloat16)
    path = tmp_path / "table.bin"
    with open(path, "wb") as f:
        f.write(b"\0" * 128)
        f.write(table.view(torch.uint8).numpy().tobytes())
    rc = RowCache(str(path), num_rows=50, row_bytes=48, slots=4, file_offset=128)
    assert torch.equal(rc.gather([3, 7, 3, 49]), table[[3, 7, 3, 49]])
    assert rc.stats == {"hits": 1, "misses": 3, "evictions": 0, "read_errors": 0} and rc.check_invariant()
    assert torch.equal(rc.gather([10, 11]), table[[10, 11]])            # one free slot, one eviction
    assert rc.stats["evictions"] == 1 and rc.check_invariant()
    # a batch with more distinct rows than slots cannot be pinned at once
    with pytest.raises(MemoryError):
        rc.resolve([20, 21, 22, 23, 24])
    assert rc.check_invariant()
    rc.end_batch()
    with pytest.raises(IndexError):
        rc.resolve([50])
    # a failing read leaves the maps consistent
    rc._read_row = lambda row: (_ for _ in ()).throw(IOError("injected"))
    with pytest.raises(IOError):
        rc.resolve([30])
    assert rc.check_invariant() and rc.stats["read_errors"] == 1
    rc.close()


def test_probe_reports_and_recommends(tmp_path):
    from metrale_inference_alpha_b200.storage.probe import decide, run_probe
    rep = run_probe(str(tmp_path / "probe"), blocks=8, block_kib=64)
    assert rep["dir_writable"] and "read_gbs" in rep["buffered"] and rep["recommendation"] in ("file", "file-direct")
    assert decide({"dir_writable": False}) == "memory"
    assert decide({"dir_writable": True, "buffered": {"read_gbs": 2.0}, "direct": {"error": "x"}}) == "file"
    assert decide({"dir_writable": True, "buffered": {"read_gbs": 2.0}, "direct": {"read_gbs": 3.0}}) == "file-direct"


# ----------------------------------------------------------------------------- KV tier under the prefix cache
@pytest.mark.parametrize("use_files", [False, True])
def test_evicted_prefix_blocks_come_back_from_the_tier(tmp_path, use_files):
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    sp = SamplingParams(max_tokens=4, temperature=0.0)
    common = dict(model="tiny-dense", device="cpu", max_num_seqs=2, max_model_len=256, num_kv_blocks=14)
    plain = LLMEngine(EngineArgs(**common))
    tiered = LLMEngine(EngineArgs(**common, kv_tier_blocks=64, kv_tier_dir=str(tmp_path / "tier") if use_files else None,
                                  kv_tier_host_blocks=4 if use_files else 0))
    a = list(range(10, 10 + 100))                              # 6 full blocks of 16
    others = [list(range(300 + 150 * i, 300 + 150 * i + 120)) for i in range(3)]
    want_a = plain.generate([a], sp)[0].output_ids
    first = tiered.generate([a], sp)[0]
    assert first.output_ids == want_a and first.cached_tokens == 0
    for o in others:                                           # push a's blocks out of the 13-block pool
        tiered.generate([o], sp)
    st = tiered.prefix.stats()
    assert st["tier_stored"] >= 6
    again = tiered.generate([a], sp)[0]
    assert again.output_ids == want_a
    assert again.cached_tokens >= 80                           # restored from the tier, not recomputed
    st = tiered.prefix.stats()
    assert st["tier_hits"] >= 1 and st["tier_restored"] >= 5 and st["tier_hit_tokens"] >= 80
    # the plain engine recomputes the same prompt from scratch after the same churn
    for o in others:
        plain.generate([o], sp)
    assert plain.generate([a], sp)[0].cached_tokens < again.cached_tokens
    # a different namespace (adapter) never sees these records
    from metrale_inference_alpha_b200.cache.kv_tier import chain_digest
    assert chain_digest(b"", a[:16], None) != chain_digest(b"", a[:16], "adapter-x")


def test_tier_capacity_overwrites_the_least_recently_used_record():
    from metrale_inference_alpha_b200.cache import KvCacheConfig, PagedKvCache
    from metrale_inference_alpha_b200.cache.kv_tier import KvTierStore
    kv = PagedKvCache(KvCacheConfig(2, 2, 16, block_size=4), 8)
    for i in range(8):
        for L in range(2):
            kv.k[L][i].fill_(i + L)
            kv.v[L][i].fill_(-(i + L))
    st = KvTierStore(kv, capacity_blocks=2)
    st.put(b"a", 1)
    st.put(b"b", 2)
    st.put(b"a", 1)                                            # refresh: b is now the oldest
    st.put(b"c", 3)
    assert st.has(b"a") and st.has(b"c") and not st.has(b"b") and st.stats["overwritten"] == 1
    assert st.restore(b"c", 5) and not st.restore(b"b", 6)
    assert torch.equal(kv.k[1][5], kv.k[1][3]) and torch.equal(kv.v[0][5], kv.v[0][3])


def test_kv_tier_is_refused_for_recurrent_models():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    with pytest.raises(ValueError):
        LLMEngine(EngineArgs(model="tiny-hybrid-moe", device="cpu", num_kv_blocks=32, kv_tier_blocks=8))


def test_nvfp4_tier_records_are_a_third_of_the_bytes_and_restore_within_the_formats_noise():
    from metrale_inference_alpha_b200.cache import KvCacheConfig, PagedKvCache
    from metrale_inference_alpha_b200.cache.kv_tier import KvTierStore
    kv = PagedKvCache(KvCacheConfig(2, 2, 64, block_size=4), 8)
    g = torch.Generator().manual_seed(0)
    for L in range(2):
        kv.k[L].copy_(torch.randn(kv.k[L].shape, generator=g).to(kv.k[L].dtype))
        kv.v[L].copy_(torch.randn(kv.v[L].shape, generator=g).to(kv.v[L].dtype))
    st = KvTierStore(kv, capacity_blocks=4, codec="nvfp4")
    elem = kv.k[0].element_size()
    rows = 2 * 2 * 4 * 2                                       # layers x (k, v) x tokens x kv heads
    assert st.record_bytes == rows * (32 + 4 + 4) and st.raw_bytes == rows * 64 * elem
    want_k, want_v = kv.k[1][3].clone().float(), kv.v[0][3].clone().float()
    st.put(b"x", 3)
    assert st.restore(b"x", 6)
    for got, want in ((kv.k[1][6].float(), want_k), (kv.v[0][6].float(), want_v)):
        rel = float((got - want).norm() / want.norm())
        assert 0.0 < rel < 0.15, rel                           # 4-bit values with a scale per 16 channels
    with pytest.raises(ValueError):
        KvTierStore(kv, capacity_blocks=4, codec="int3")


@pytest.mark.parametrize("name,row_bytes,bound", [("nvfp4", 76, 0.12), ("turbo4", 68, 0.12), ("turbo3", 52, 0.22), ("turbo2", 36, 0.40)])
def test_tier_codecs_meet_their_sizes_and_distortion_with_an_outlier_channel(name, row_bytes, bound):
    """The Lloyd-Max distortion of a unit Gaussian is 0.0095 / 0.0345 / 0.1175 at 4 / 3 / 2 bits (relative rms error
    0.097 / 0.186 / 0.343); the Walsh-Hadamard rotation is what makes a row with one channel 20 x the rest meet it."""
    from metrale_inference_alpha_b200.cache.kv_codec import fwht, make_codec, roundtrip
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 128, generator=g)
    x[:, 5] *= 20
    assert torch.allclose(fwht(fwht(x, 128), 128), x, atol=1e-4)
    y, b = roundtrip(make_codec(name), x)
    assert b == row_bytes and float((y - x).norm() / x.norm()) < bound
    # a latent row of 576 channels (not a power of two): the rotation runs over blocks of 64
    z = torch.randn(8, 576, generator=g)
    y, b = roundtrip(make_codec(name), z)
    assert float((y - z).norm() / z.norm()) < bound
    # an all-zero row stays zero
    y, _ = roundtrip(make_codec(name), torch.zeros(2, 64))
    assert float(y.abs().max()) == 0.0


@pytest.mark.parametrize("codec", ["turbo4", "turbo2"])
def test_tier_store_round_trips_blocks_through_a_turbo_codec(codec):
    from metrale_inference_alpha_b200.cache import KvCacheConfig, PagedKvCache
    from metrale_inference_alpha_b200.cache.kv_tier import KvTierStore
    kv = PagedKvCache(KvCacheConfig(2, 2, 64, block_size=4), 8)
    g = torch.Generator().manual_seed(1)
    for L in range(2):
        kv.k[L].copy_(torch.randn(kv.k[L].shape, generator=g).to(kv.k[L].dtype))
        kv.v[L].copy_(torch.randn(kv.v[L].shape, generator=g).to(kv.v[L].dtype))
    st = KvTierStore(kv, capacity_blocks=2, codec=codec)
    want = kv.v[1][2].clone().float()
    st.put(b"k", 2)
    assert st.restore(b"k", 7)
    rel = float((kv.v[1][7].float() - want).norm() / want.norm())
    assert 0.0 < rel < (0.12 if codec == "turbo4" else 0.40)
    assert st.record_bytes == 2 * 2 * 4 * 2 * (64 * int(codec[-1]) // 8 + 4)


def test_engine_serves_prefix_hits_from_an_nvfp4_tier(tmp_path):
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    sp = SamplingParams(max_tokens=4, temperature=0.0)
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=2, max_model_len=256, num_kv_blocks=14,
                               kv_tier_blocks=64, kv_tier_codec="nvfp4"))
    a = list(range(10, 10 + 100))
    eng.generate([a], sp)
    for i in range(3):
        eng.generate([list(range(300 + 150 * i, 300 + 150 * i + 120))], sp)
    again = eng.generate([a], sp)[0]
    st = eng.prefix.stats()
    assert again.cached_tokens >= 80 and len(again.output_ids) == 4 and st["tier_restored"] >= 5
    assert eng.kv_tier.record_bytes * 3 < eng.kv_tier.raw_bytes            # 76 bytes per 128 channels against 256 (bf16) or 512
    eng.close()
