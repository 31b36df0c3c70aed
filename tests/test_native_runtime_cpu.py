"""The C++ host runtime against its Python oracles: randomized differential tests of the block
allocator and radix prefix index, the JSON recogniser and token-mask fill, and the parallel file
reader. Mirrors the reference's unit tests of ``crates/cache`` and ``crates/grammar``."""
import json
import os
import random

import pytest
import torch

from metrale_inference_alpha_b200 import native
from metrale_inference_alpha_b200.cache.block_pool import BlockAllocator, NoFreeBlocks
from metrale_inference_alpha_b200.cache.radix import RadixTree
from metrale_inference_alpha_b200.server.grammar import JsonMatcher
from metrale_inference_alpha_b200.server.tokenizer import ByteTokenizer

pytestmark = pytest.mark.skipif(not native.available(), reason="native host runtime not built")


def test_allocator_matches_python_oracle_under_random_traffic():
    rng = random.Random(1)
    a, b = BlockAllocator(64), native.NativeBlockAllocator(64)
    held = []
    for _ in range(2000):
        op = rng.random()
        if op < 0.45:
            n = rng.randint(1, 5)
            try:
                x = a.alloc(n)
            except NoFreeBlocks:
                with pytest.raises(NoFreeBlocks):
                    b.alloc(n)
                continue
            assert b.alloc(n) == x
            held += [[blk] for blk in x]
        elif op < 0.6 and held:
            h = rng.choice(held)
            a.incref(h)
            b.incref(h)
            held.append(list(h))
        elif held:
            h = held.pop(rng.randrange(len(held)))
            assert a.free(h) == b.free(h)
        assert a.num_free == b.num_free and a.num_used == b.num_used
    for blk in range(64):
        assert a.refcount[blk] == b.refcount[blk]
    with pytest.raises(AssertionError):
        b.free([5]) if b.refcount[5] == 0 else (_ for _ in ()).throw(AssertionError())


def test_radix_matches_python_oracle_under_random_traffic():
    rng = random.Random(2)
    bs = 4
    pa, na = BlockAllocator(256), native.NativeBlockAllocator(256)
    evp, evn = [], []
    pt = RadixTree(pa, bs, needs_snapshot=False, on_snapshot_evict=evp.append)
    nt = native.NativeRadixTree(na, bs, needs_snapshot=False, on_snapshot_evict=evn.append)
    live = []
    vocab = 6                                    # small alphabet: many shared prefixes
    for step in range(1500):
        op = rng.random()
        toks = [rng.randrange(vocab) for _ in range(rng.randint(1, 30))]
        adapter = rng.choice([None, None, "a", "b"])
        if op < 0.4:
            mp, mn = pt.match(toks, adapter), nt.match(toks, adapter)
            assert (mp.blocks, mp.tokens, mp.snapshot) == (mn.blocks, mn.tokens, mn.snapshot)
            live.append(mp.blocks)
        elif op < 0.75:
            nblk = len(toks) // bs
            if nblk == 0 or pa.num_free < nblk:
                continue
            bp, bn = pa.alloc(nblk), na.alloc(nblk)
            assert bp == bn
            snaps = {bs * rng.randint(1, nblk): step} if rng.random() < 0.3 else None
            assert pt.insert(toks, bp, adapter, snaps) == nt.insert(toks, bn, adapter, snaps)
            pa.free(bp)
            na.free(bn)
        elif op < 0.9 and live:
            h = live.pop(rng.randrange(len(live)))
            pa.free(h)
            na.free(h)
        else:
            k = rng.randint(1, 6)
            assert pt.evict(k) == nt.evict(k)
        assert pa.num_free == na.num_free, step
        assert pt.stats() == nt.stats()
        assert pt.evictable_blocks() == nt.evictable_blocks()
    assert sorted(evp) == sorted(evn)
    pt.clear()
    nt.clear()
    for h in live:
        pa.free(h)
        na.free(h)
    assert pa.num_used == na.num_used == 0


def test_radix_snapshot_gate_matches_oracle():
    pa, na = BlockAllocator(32), native.NativeBlockAllocator(32)
    pt, nt = RadixTree(pa, 4, needs_snapshot=True), native.NativeRadixTree(na, 4, needs_snapshot=True)
    toks = list(range(1, 14))
    pt.insert(toks, pa.alloc(3), snapshots={8: 5})
    nt.insert(toks, na.alloc(3), snapshots={8: 5})
    mp, mn = pt.match(toks), nt.match(toks)
    assert (mn.blocks, mn.tokens, mn.snapshot) == (mp.blocks, mp.tokens, mp.snapshot) == (mp.blocks, 8, 5)


DOCS = ['{"a": 1, "b": [true, null, -2.5e3], "c": {"d": "x\\n\\u00e9"}}', '  {"k": ""}  ', '{}', '{"a": 01}',
        '{"a": 1,}', '{a: 1}', '{"a": tru}', '{"a": "x}', '[1, 2]', '{"a": [], "b": {}}', '{"a": -}', '{"a": 1.}',
        '{"a": 1e}', '{"a": 1e+5, "b": 0.25, "c": -0}', '{"a": [1,, 2]}', '{"a": "\\q"}', '{"a": "\\u12g4"}']


@pytest.mark.parametrize("doc", DOCS)
def test_json_recogniser_agrees_with_json_loads(doc):
    g = native.NativeJsonGrammar(ByteTokenizer(512), eos_token_id=0)
    ok = g.feed_bytes(doc.encode()) and g.is_complete()
    try:
        expect = isinstance(json.loads(doc), dict)
    except ValueError:
        expect = False
    assert ok == expect


def test_every_prefix_of_a_valid_document_is_accepted_and_python_matcher_agrees():
    doc = '{"name": "x", "n": [1, 2.5, -3e-2, {"t": true, "f": false, "z": null}], "s": "a\\"b"}'.encode()
    for i in range(1, len(doc) + 1):
        g = native.NativeJsonGrammar(ByteTokenizer(512), eos_token_id=0)
        assert g.feed_bytes(doc[:i]), doc[:i]
        m = JsonMatcher(require_object=True)
        assert m.feed_bytes(doc[:i])
        assert g.is_complete() == m.is_complete() == (i == len(doc))


def test_token_mask_is_exact_and_drives_generation_to_valid_json():
    tk = ByteTokenizer(512)
    g = native.NativeJsonGrammar(tk, eos_token_id=0)
    m0 = g.allowed_mask(512)
    legal = {t for t in range(512) if m0[t]}
    assert legal == {tk.encode(c)[0] for c in ' \t\n\r{'}      # only whitespace or '{' may start an object
    gen = torch.Generator().manual_seed(5)
    out = []
    for _ in range(300):
        logits = torch.randn(512, generator=gen)
        if len(out) > 30:
            logits[0] += 50.0
            logits[tk.encode("}")[0]] += 20.0
            logits[tk.encode('"')[0]] += 10.0
        mask = g.allowed_mask(512)
        t = int(torch.where(mask, logits, torch.full_like(logits, -1e30)).argmax())
        if t == 0:
            break
        g.advance(t)
        out.append(t)
    assert isinstance(json.loads(tk.decode(out)), dict)
    import pickle
    g2 = pickle.loads(pickle.dumps(g))                          # travels to follower ranks by replay
    assert g2.is_complete() and torch.equal(g2.allowed_mask(512), g.allowed_mask(512))


def test_mask_fill_over_a_large_vocabulary_is_fast():
    import time

    class Tok:
        vocab_size = 150_000

        def token_bytes(self, t):
            rng = random.Random(t)
            return bytes(rng.choice(b'abcdefghij {}[]":,0123456789') for _ in range(rng.randint(1, 8)))
    g = native.NativeJsonGrammar(Tok(), eos_token_id=None)
    g.feed_bytes(b'{"key": ')
    g.allowed_mask(150_000)
    t0 = time.perf_counter()
    for _ in range(5):
        mask = g.allowed_mask(150_000)
    dt = (time.perf_counter() - t0) / 5
    assert mask.any() and dt < 0.05, dt


def test_parallel_reader_plain_and_direct(tmp_path):
    path = tmp_path / "blob.bin"
    data = os.urandom(3 * (8 << 20) + 12345)
    path.write_bytes(data)
    ranges = [(0, 100), (4096, 8 << 20), (5000, 777), ((8 << 20) + 13, (16 << 20) + 1000), (len(data) - 50, 50)]
    for direct in (False, True):
        bufs = [torch.zeros(n, dtype=torch.uint8) for _, n in ranges]
        total = native.read_ranges(str(path), [o for o, _ in ranges], [n for _, n in ranges],
                                   [b.data_ptr() for b in bufs], threads=4, direct=direct)
        assert total == sum(n for _, n in ranges)
        for (o, n), b in zip(ranges, bufs):
            assert bytes(b.numpy().tobytes()) == data[o:o + n]
    with pytest.raises(OSError):
        native.read_ranges(str(tmp_path / "missing"), [0], [1], [bufs[0].data_ptr()])
    with pytest.raises(OSError):
        native.read_ranges(str(path), [len(data) - 10], [100], [bufs[1].data_ptr()])     # past the end


def test_fast_checkpoint_source_reads_the_same_tensors_as_safetensors(tmp_path):
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.weights.fast_source import FastSafetensorsSource
    from metrale_inference_alpha_b200.weights.source import SafetensorsSource, SyntheticSource, write_checkpoint
    cfg = preset("tiny-dense")
    write_checkpoint(SyntheticSource(cfg, seed=3), cfg, tmp_path)
    slow, fast = SafetensorsSource(tmp_path), FastSafetensorsSource(tmp_path, threads=3)
    names = sorted(slow.names())
    assert names == sorted(fast.names()) and names
    fast.prefetch(names[: len(names) // 2])                 # one batched read, the rest on demand
    for n in names:
        a, b = slow.get(n), fast.get(n)
        assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b), n
    assert fast.bytes_read > 0


def test_engine_loads_a_checkpoint_directory_through_the_fast_reader(tmp_path):
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.weights.source import SyntheticSource, write_checkpoint
    cfg = preset("tiny-dense")
    write_checkpoint(SyntheticSource(cfg, seed=0), cfg, tmp_path)
    a = LLMEngine(EngineArgs(model=str(tmp_path), device="cpu", max_model_len=128))
    b = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_model_len=128, seed=0))
    p = [[1, 2, 3, 4, 5]]
    sp = SamplingParams(max_tokens=6)
    assert a.generate(p, sp)[0].output_ids == b.generate(p, sp)[0].output_ids


def test_loader_reads_modelopt_input_scale():
    """A ModelOpt NVFP4 checkpoint's `<linear>.input_scale` becomes the static activation scale of
    the down and o projections; linears without one stay on dynamic scales (0)."""
    import torch
    from metrale_inference_alpha_b200.config.model_config import tiny_dense
    from metrale_inference_alpha_b200.weights.loader import load_weights
    from metrale_inference_alpha_b200.weights.source import DictSource, SyntheticSource
    cfg = tiny_dense(weight_format="nvfp4")
    syn = SyntheticSource(cfg, seed=0)
    t = {n: syn.get(n) for n in syn.names()}
    t["model.layers.0.mlp.down_proj.input_scale"] = torch.tensor(0.00125)
    t["model.layers.0.self_attn.o_proj.input_scale"] = torch.tensor([0.0025])
    t["model.layers.1.mlp.down_proj.input_scale"] = torch.tensor(float("nan"))
    w = load_weights(cfg, DictSource(t, syn.quant_config))
    assert abs(w.layers[0].ffn.down_in_scale - 0.00125) < 1e-9
    assert abs(w.layers[0].mixer.o_in_scale - 0.0025) < 1e-9
    assert w.layers[1].ffn.down_in_scale == 0.0 and w.layers[1].mixer.o_in_scale == 0.0
