"""Config-1 plumbing check on CPU: the engine (scheduler + paged KV + prefix cache + sampler)
must reproduce, token for token and logit for logit, a straight-line oracle that re-runs the
whole sequence through the decoder without any cache reuse."""
import pytest
import torch

from metrale_inference_alpha_b200.cache import KvCacheConfig, PagedKvCache
from metrale_inference_alpha_b200.config.model_config import preset
from metrale_inference_alpha_b200.engine.batch import ForwardBatch
from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.models.decoder import Decoder, LayerCaches
from metrale_inference_alpha_b200.sampling.params import SamplingParams


def _oracle_greedy(engine, prompt, n):
    """Re-prefill the whole sequence from scratch for every new token."""
    cfg = engine.cfg
    dec = Decoder(cfg, engine.weights)
    toks = list(prompt)
    logits_hist = []
    for _ in range(n):
        kv = PagedKvCache(KvCacheConfig(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), 64)
        nb = (len(toks) + 15) // 16
        b = ForwardBatch.build([dict(tokens=toks, start_pos=0, blocks=list(range(1, nb + 1)))], 16)
        lg, _ = dec.forward(b, LayerCaches(cfg, kv=kv))
        logits_hist.append(lg[0].float())
        toks.append(int(lg[0].float().argmax()))
    return toks[len(prompt):], logits_hist


def test_tiny_dense_engine_matches_oracle():
    g = torch.Generator().manual_seed(42)
    prompts = [torch.randint(0, 4096, (32,), generator=g).tolist() for _ in range(4)]
    eng = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=256, num_kv_blocks=128, max_prefill_tokens=48))
    outs = eng.generate(prompts, SamplingParams(max_tokens=24, temperature=0.0))
    assert len(outs) == 4
    for p, o in zip(prompts, outs):
        want, _ = _oracle_greedy(eng, p, 24)
        assert o.output_ids == want
        assert o.finish_reason == "length"
    st = eng.stats()
    assert st["finished"] == 4 and st["free_blocks"] + st.get("prefix_cache", {}).get("nodes", 0) == 127


def test_prefix_cache_hit_gives_same_tokens():
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 4096, (48,), generator=g).tolist()
    eng = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=256, num_kv_blocks=128))
    a = eng.generate([shared + [5, 6, 7]], SamplingParams(max_tokens=8))[0]
    b = eng.generate([shared + [5, 6, 7]], SamplingParams(max_tokens=8))[0]
    assert a.output_ids == b.output_ids
    assert a.cached_tokens == 0 and b.cached_tokens == 48
    eng2 = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=256, num_kv_blocks=128,
                                enable_prefix_caching=False))
    c = eng2.generate([shared + [5, 6, 7]], SamplingParams(max_tokens=8))[0]
    assert c.output_ids == a.output_ids


def test_sampling_is_seeded_and_batch_invariant():
    g = torch.Generator().manual_seed(2)
    p1 = torch.randint(0, 4096, (20,), generator=g).tolist()
    p2 = torch.randint(0, 4096, (33,), generator=g).tolist()
    sp = SamplingParams(max_tokens=12, temperature=0.8, top_k=40, top_p=0.95, seed=123)
    eng = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=256, num_kv_blocks=128,
                               enable_prefix_caching=False))
    alone = eng.generate([p1], sp)[0].output_ids
    together = eng.generate([p1, p2], [sp, SamplingParams(max_tokens=5)])[0].output_ids
    assert alone == together


def test_quantised_tiny_models_run_end_to_end():
    for fmt in ("nvfp4", "fp8_row"):
        eng = LLMEngine(EngineArgs(model=preset("tiny-dense", weight_format=fmt, kv_dtype="fp8"),
                                   max_model_len=128, num_kv_blocks=64))
        out = eng.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=6))[0]
        assert len(out.output_ids) == 6


def test_penalties_and_logit_bias_path():
    eng = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=128, num_kv_blocks=64))
    base = eng.generate([[9, 8, 7, 6]], SamplingParams(max_tokens=6))[0].output_ids
    forced = eng.generate([[9, 8, 7, 6]], SamplingParams(max_tokens=6, logit_bias={77: 100.0}))[0].output_ids
    assert forced == [77] * 6
    rep = eng.generate([[9, 8, 7, 6]], SamplingParams(max_tokens=6, repetition_penalty=1.5,
                                                      frequency_penalty=0.5))[0].output_ids
    assert len(rep) == 6 and isinstance(base, list)


def test_swap_preemption_resumes_without_recompute_and_matches_recompute_mode(tmp_path):
    """Under KV pressure the swap mode copies a victim's blocks out and back; tokens must equal
    both the roomy run and the recompute mode, and no prompt token is prefetched twice."""
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    prompts = [[(7 * i + j) % 200 + 1 for j in range(40)] for i in range(4)]
    sp = SamplingParams(max_tokens=40)

    def run(**kw):
        eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=128,
                                   enable_prefix_caching=False, use_cuda_graphs=False, **kw))
        eng.sched_cfg.decode_reserve_tokens = 0
        outs = eng.generate(prompts, sp)
        return [o.output_ids for o in outs], eng
    roomy, _ = run(num_kv_blocks=64)
    swap, e1 = run(num_kv_blocks=14, preempt_mode="swap", swap_space_bytes=1 << 20, swap_dir=str(tmp_path))
    rec, e2 = run(num_kv_blocks=14)
    assert swap == roomy == rec
    assert e1.scheduler.stats["preempted"] > 0 and e1.spill.stats["saved"] > 0
    assert e1.spill.stats["saved"] == e1.spill.stats["restored"]
    assert e1.scheduler.stats["prefill_tokens"] == 4 * 40            # nothing was prefetched again
    assert e2.scheduler.stats["prefill_tokens"] > 4 * 40             # recompute mode re-ran prompts
    # a tiny host budget pushes victims to swap files
    disk, e3 = run(num_kv_blocks=14, preempt_mode="swap", swap_space_bytes=1, swap_dir=str(tmp_path))
    assert disk == roomy and e3.spill.stats["to_disk"] > 0 and not list(tmp_path.glob("*.pt"))


def test_dry_and_lz_penalties_tables_and_effect_on_generation():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.host import dry_penalties, lz_penalty
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    toks = [1, 2, 3, 4, 9, 1, 2, 3]                     # "... 1 2 3" seen before, followed by 4
    pen = dry_penalties(toks, multiplier=0.8, base=2.0, allowed=2, window=64)
    assert pen == {4: 0.8 * 2.0 ** (3 - 2)}              # repeat of length 3 would be extended by token 4
    assert dry_penalties(toks, 0.8, 2.0, allowed=4, window=64) == {}
    assert dry_penalties(toks, 0.0, 2.0, 2, 64) == {}
    loop = [5, 6, 7, 8] * 3
    assert lz_penalty(loop, 0.5) == {5: 0.5 * 8}         # suffix of length 8 matched; next would be 5
    assert lz_penalty([1, 2, 3], 0.5) == {}
    # a greedy random model falls into a loop quickly; DRY must break exact repetition
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_model_len=256))
    prompt = [3, 4, 5, 6]
    plain = eng.generate([prompt], SamplingParams(max_tokens=60))[0].output_ids
    dry = eng.generate([prompt], SamplingParams(max_tokens=60, dry_multiplier=4.0, dry_base=2.0))[0].output_ids

    def longest_repeat(x):
        best = 0
        for i in range(len(x)):
            for j in range(i + 1, len(x)):
                k = 0
                while j + k < len(x) and x[i + k] == x[j + k]:
                    k += 1
                best = max(best, k)
        return best
    assert longest_repeat(dry) <= longest_repeat(plain)
    assert longest_repeat(dry) < 12


def test_kv_high_precision_layers_mix_dtypes_per_layer():
    from metrale_inference_alpha_b200.cache import KvCacheConfig
    from metrale_inference_alpha_b200.engine.llm_engine import parse_layer_list
    assert parse_layer_list("first:2,last:1,5", 8) == (0, 1, 5, 7)
    import pytest as _pt
    with _pt.raises(ValueError):
        parse_layer_list("9", 8)
    plain = KvCacheConfig(4, 2, 64, 16, "fp8")
    mixed = KvCacheConfig(4, 2, 64, 16, "fp8", high_precision_layers=(0, 3))
    assert mixed.block_bytes() == plain.block_bytes() * 6 // 4             # two of four layers at 2 bytes
    assert KvCacheConfig(4, 2, 64, 16, "bf16", high_precision_layers=(0,)).block_bytes() == 2 * plain.block_bytes()
    eng = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=128, num_kv_blocks=32, kv_cache_dtype="fp8",
                               kv_high_precision_layers="first:1"))
    kv = eng.runner.kv
    assert kv.k[0].dtype == torch.bfloat16 and kv.k[1].dtype == torch.uint8 and kv.v[0].dtype == torch.bfloat16
    prompts = [list(range(5, 40))]
    hp = eng.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0))[0].output_ids
    all_bf16 = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=128, num_kv_blocks=32)).generate(
        prompts, SamplingParams(max_tokens=8, temperature=0.0))[0].output_ids
    assert len(hp) == 8 and len(all_bf16) == 8


def test_seeded_temperature_request_is_unchanged_by_speculation():
    """Drafts are verified by argmax, so only greedy requests get them: a seeded temperature
    request decodes the same tokens with speculation on and off, also when it shares steps with
    greedy requests that do speculate."""
    prompts = [[3, 4, 5, 6, 3, 4, 5, 6, 3, 4, 5, 6, 3, 4], [9, 8, 7, 9, 8, 7, 9, 8, 7, 9, 8]]
    params = [SamplingParams(max_tokens=16, temperature=0.9, top_p=0.95, seed=1234),
              SamplingParams(max_tokens=16, temperature=0.0)]
    outs = {}
    for spec in ("none", "ngram"):
        eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=256,
                                   speculative=spec, num_drafts=3, mtp_gate=False))
        outs[spec] = [o.output_ids for o in eng.generate(prompts, params)]
    assert outs["ngram"] == outs["none"]


def test_a_reported_device_status_latches_the_engine_fault():
    """The status word comes back with the sampled ids; a non-zero value (an expired bounded
    wait, a skipped out-of-range access) raises, and step() turns it into a latched fault."""
    from metrale_inference_alpha_b200.ops._native import KernelError
    from metrale_inference_alpha_b200.scheduler.types import FatalDeviceError
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_model_len=128, num_kv_blocks=32))
    r = eng.runner
    r.host_status[0] = 0x400                               # what MB_ST_TIMEOUT_PEER looks like on the host
    r.status_pending = True
    with pytest.raises(KernelError, match="device status 0x400"):
        r._check_status()
    assert not r.status_pending
    eng.add_request([1, 2, 3], SamplingParams(max_tokens=4))
    real = r._check_status

    def reported():
        r.host_status[0] = 0x500
        r.status_pending = True
        real()
    r._check_status = reported
    r._post_status = lambda: None
    execute = r._execute

    def execute_and_check(plan):
        out = execute(plan)
        r._check_status()
        return out
    r._execute = execute_and_check
    with pytest.raises(FatalDeviceError):
        eng.step()
    assert eng.fault.is_set()
    with pytest.raises(FatalDeviceError):
        eng.add_request([1], SamplingParams(max_tokens=1))


@pytest.mark.parametrize("model", ["tiny-nemotron-h", "tiny-hybrid-moe"])
def test_recurrent_models_reuse_a_prompt_prefix_through_a_state_snapshot(model):
    """A prompt seen before resumes from the state snapshot taken at its last full block
    (prefill stops there once, so that the snapshot exists): the second request computes less
    than one block of prompt tokens and produces the same tokens."""
    eng = LLMEngine(EngineArgs(model=preset(model), device="cpu", max_num_seqs=4, max_model_len=512))
    prompt = [(7 * j) % 300 + 1 for j in range(300)]
    cold = eng.generate([prompt], SamplingParams(max_tokens=6))[0]
    warm = eng.generate([prompt], SamplingParams(max_tokens=6))[0]
    longer = eng.generate([prompt + [5, 6, 7]], SamplingParams(max_tokens=4))[0]
    assert cold.cached_tokens == 0
    assert warm.cached_tokens == 288 and warm.output_ids == cold.output_ids
    assert longer.cached_tokens == 288


def test_config1_tiny_dense_64_tokens_per_step_logits_against_an_independent_restatement():
    """The plumbing configuration end to end: 4 requests of 32 uniform-random token ids (seed 42),
    greedy decode of 64 tokens, paged KV with block 16, weights N(0, 0.02) from seed 0. Every
    decode step's logits and every token are compared with an independent fp32 restatement of
    the architecture (plain tensor algebra over the whole sequence, no cache, no engine code)."""
    from metrale_inference_alpha_b200.weights.source import SyntheticSource
    from tests.test_families_cpu import _oracle_logits
    cfg = preset("tiny-dense")
    hf = dict(model_type="qwen3", num_attention_heads=cfg.num_heads, num_key_value_heads=cfg.num_kv_heads,
              head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_eps, num_hidden_layers=cfg.num_layers, rope_theta=cfg.rope_theta)
    syn = SyntheticSource(cfg, seed=0)
    canon = {n: syn.get(n) for n in syn.names()}
    if cfg.tie_embeddings and "lm_head.weight" not in canon:
        canon["lm_head.weight"] = canon["model.embed_tokens.weight"]
    g = torch.Generator().manual_seed(42)
    prompts = [torch.randint(0, cfg.vocab_size, (32,), generator=g).tolist() for _ in range(4)]
    eng = LLMEngine(EngineArgs(model=cfg, device="cpu", seed=0, max_model_len=128, num_kv_blocks=64, block_size=16))
    steps = []                                             # (positions of the logit rows, logits) per forward
    inner = eng.runner._forward_select

    def capture(batch, greedy, want_lp, n_rows, feed=False):
        lg = inner(batch, greedy, want_lp, n_rows, feed)
        steps.append((batch.positions[batch.logit_rows].tolist(), batch.q_start.tolist(), lg.float().clone()))
        return lg
    eng.runner._forward_select = capture
    outs = eng.generate(prompts, SamplingParams(max_tokens=64, temperature=0.0))
    assert [len(o.output_ids) for o in outs] == [64] * 4
    checked = flips = 0
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in range(64):
            want = _oracle_logits(hf, lambda n: canon[n], lambda n: n in canon, toks)
            if int(want.argmax()) != o.output_ids[t]:
                # the engine rounds the residual stream to bf16 where the restatement keeps fp32: only a
                # near-tie of the restatement's own logits may resolve differently
                gap = (want.max() - want[o.output_ids[t]]).item()
                assert gap < 1e-2 * want.abs().max().item(), (t, int(want.argmax()), o.output_ids[t], gap)
                flips += 1
            toks.append(o.output_ids[t])
    # per-step logits: every forward's rows against the restatement at the same position of the same request
    seqs = {i: list(p) + o.output_ids for i, (p, o) in enumerate(zip(prompts, outs))}
    for pos_rows, _, lg in steps:
        if len(pos_rows) != 4:
            continue                                        # (prefill steps of fewer requests are covered by the token check)
        for i, pos in enumerate(pos_rows):
            want = _oracle_logits(hf, lambda n: canon[n], lambda n: n in canon, seqs[i][:pos + 1])
            err = (lg[i] - want).abs().max().item()
            assert err < 2e-2 * want.abs().max().item() + 2e-3, (pos, err)
            checked += 1
        if checked >= 4 * 16:
            break                                           # 16 full decode steps of logits (the rest by tokens)
    assert checked >= 4 * 16
    assert flips <= 4                                       # of 256 tokens


@pytest.mark.parametrize("model", ["tiny-hybrid-moe", "tiny-nemotron-h", "tiny-dense"])
def test_rollback_to_a_ring_snapshot_resumes_exactly(model):
    """Generate, roll the request back to an earlier length, continue: greedy decoding must
    reproduce the tokens it produced the first time (recurrent state restored from the decode
    ring, attention KV simply rewritten). A length with no ring snapshot is declined on recurrent
    models and the sequence is left untouched."""
    eng = LLMEngine(EngineArgs(model=preset(model), device="cpu", max_num_seqs=2, max_model_len=256,
                               decode_rollback_ring=3, decode_rollback_interval=4, enable_prefix_caching=False))
    rid = eng.add_request([5, 6, 7, 8, 9, 10, 11], SamplingParams(max_tokens=24))
    first = None
    while eng.has_work():
        outs = eng.step()
        seq = next((s for s in eng.scheduler.running if s.req.request_id == rid), None)
        if seq is not None and seq.num_output == 14 and first is None:
            first = list(seq.tokens[seq.prompt_len:])
            recurrent = eng.runner.pool is not None
            if recurrent:
                assert eng.scheduler.rollback_positions(seq) == [4, 8, 12]
                assert not eng.rollback_request(rid, 7)          # no snapshot at 7
                assert list(seq.tokens[seq.prompt_len:]) == first
            assert eng.rollback_request(rid, 8)
            assert seq.num_output == 8
        final = [o for o in outs if o.finished]
    assert first is not None and final
    assert final[0].output_ids[:14] == first
    assert len(final[0].output_ids) == 24


def test_close_is_ordered_idempotent_and_final(tmp_path):
    from metrale_inference_alpha_b200.scheduler.types import FatalDeviceError
    eng = LLMEngine(EngineArgs(model="tiny-dense", max_model_len=256, num_kv_blocks=32, kv_tier_blocks=8, kv_tier_dir=str(tmp_path / "t")))
    eng.generate([[5, 6, 7, 8] * 6], SamplingParams(max_tokens=3, temperature=0.0))
    rid = eng.add_request([1, 2, 3], SamplingParams(max_tokens=50))
    used = eng.runner.kv.allocator.num_free
    eng.close()
    eng.close()
    assert not eng.scheduler.has_work() and eng.kv_tier.backend._fds == []
    assert eng.runner.kv.allocator.num_free >= used            # the prefix tree gave its blocks back
    with pytest.raises(FatalDeviceError):
        eng.add_request([1, 2, 3])
    assert rid
