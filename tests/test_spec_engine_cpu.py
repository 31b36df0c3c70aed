"""Speculative decoding through the real runner is lossless: with greedy sampling the MTP and
n-gram modes must emit exactly the tokens of plain decoding, whatever the drafts were (verify +
accept + rewind of KV / positions). Mirrors the reference's "KAT equality" checks of speculative
against non-speculative output (``crates/bench`` kat_equality, ``scheduler/mtp_step.rs`` tests)."""
import pytest

from metrale_inference_alpha_b200.config.model_config import preset
from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.sampling.params import SamplingParams

PROMPTS = [[3, 4, 5, 6, 3, 4, 5, 6, 3, 4, 5], [9, 8, 7, 9, 8, 7, 9, 8], [11, 12, 13, 14, 15]]


def _run(device, **kw):
    cfg = preset("tiny-dense", mtp_layers=1)
    eng = LLMEngine(EngineArgs(model=cfg, device=device, max_num_seqs=4, max_model_len=256, mtp_gate=False, **kw))
    outs = eng.generate(PROMPTS, SamplingParams(max_tokens=24))
    return [o.output_ids for o in outs], eng


@pytest.mark.parametrize("mode", ["ngram", "mtp"])
def test_speculative_modes_are_lossless_on_cpu(mode):
    base, _ = _run("cpu")
    spec, eng = _run("cpu", speculative=mode, num_drafts=3)
    assert spec == base
    assert eng.spec_stats.drafted > 0                     # drafts were actually verified
    assert eng.spec_stats.steps < sum(len(o) for o in base) or eng.spec_stats.accepted == 0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["ngram", "mtp"])
def test_speculative_modes_are_lossless_on_gpu(mode):
    base, _ = _run("cuda")
    spec, eng = _run("cuda", speculative=mode, num_drafts=3)
    assert spec == base
    assert eng.spec_stats.drafted > 0


@pytest.mark.gpu
def test_graphed_verify_and_mtp_propose_equal_the_eager_steps():
    """The speculative loop on a GPU runs as CUDA graphs: one graph per (rung, K) for the verify
    forward and one per (rung, k) for all k draft steps of the MTP head. Outputs, draft counts and
    acceptance must equal the step-by-step (eager) drafting and plain decoding."""
    base, _ = _run("cuda")
    cfg = preset("tiny-dense", mtp_layers=1)
    res = {}
    for graphed in (False, True):
        eng = LLMEngine(EngineArgs(model=cfg, device="cuda", max_num_seqs=4, max_model_len=256, mtp_gate=False,
                                   speculative="mtp", num_drafts=3))
        eng.runner.graph_propose = graphed
        outs = eng.generate(PROMPTS, SamplingParams(max_tokens=24))
        res[graphed] = ([o.output_ids for o in outs], eng.spec_stats.drafted, eng.spec_stats.accepted)
        keys = [k for k in eng.runner.graphs if isinstance(k, tuple) and k[0] in ("mtp", "verify")]
        assert any(k[0] == "verify" and k[2] == 3 for k in keys)
        assert any(k[0] == "mtp" for k in keys) == graphed
    assert res[True][0] == base == res[False][0]
    assert res[True][1:] == res[False][1:]


def test_grammar_masks_follow_draft_rows_and_rewind_to_the_accepted_prefix():
    """Speculative verify rows with a grammar: row j is masked from the matcher state after drafts
    1..j, and the matcher is rewound to what was accepted. Output must be a legal prefix of the
    grammar and identical to the non-speculative run."""
    from metrale_inference_alpha_b200 import grammar as G
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.server.tokenizer import load_tokenizer
    outs = {}
    for spec in ("none", "ngram"):
        eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=256,
                                   speculative=spec, num_drafts=3, mtp_gate=False))
        tok = load_tokenizer(None, eng.cfg.vocab_size)
        g = G.compile_regex(r"(ab|abc|abab| )+\.")
        prompt = tok.encode("abab abab abab abab abab abab ")          # gives the n-gram proposer something to repeat
        res = []
        for _ in range(2):
            sp = SamplingParams(max_tokens=24, temperature=0.0, grammar=G.TokenMatcher(g, tok, None))
            res.append(eng.generate([prompt], sp)[0])
        outs[spec] = [r.output_ids for r in res]
        for r in res:
            text = b"".join(tok.token_bytes(t) for t in r.output_ids)
            assert G.GrammarMatcher(g).feed_bytes(text), text
        if spec == "ngram":
            assert eng.spec_stats.drafted > 0                       # the verify path really ran
    assert outs["ngram"] == outs["none"]


def test_predicted_outputs_are_verified_losslessly_and_save_steps():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.speculative.ngram import propose_from_prediction as pfp
    assert pfp([1, 2], [1, 2, 3, 4, 5], 2) == [3, 4]                          # following the prediction
    assert pfp([1, 2, 9, 4, 5, 6], [1, 2, 3, 4, 5, 6, 7, 8], 3) == [7, 8]     # re-synchronised after an edit
    assert pfp([9, 9, 9, 9], [1, 2, 3, 4], 3) == [] and pfp([1], [], 3) == [] and pfp([1, 2], [1, 2], 3) == []
    prompt = list(range(10, 40))
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=256))
    base = eng.generate([prompt], SamplingParams(max_tokens=24, temperature=0.0))[0]
    steps0 = eng.step_count
    exact = eng.generate([prompt], SamplingParams(max_tokens=24, temperature=0.0, prediction_ids=list(base.output_ids)))[0]
    steps_exact = eng.step_count - steps0
    assert exact.output_ids == base.output_ids and exact.accepted_draft_tokens >= 16 and steps_exact <= 8
    edited = list(base.output_ids)
    edited[5] = (edited[5] + 1) % 4000                                           # the guess is wrong in one place
    steps1 = eng.step_count
    part = eng.generate([prompt], SamplingParams(max_tokens=24, temperature=0.0, prediction_ids=edited))[0]
    assert part.output_ids == base.output_ids and part.rejected_draft_tokens > 0 and part.accepted_draft_tokens > 0
    assert eng.step_count - steps1 < 24
    sampled = eng.generate([prompt], SamplingParams(max_tokens=8, temperature=0.9, seed=1, prediction_ids=edited))[0]
    assert sampled.accepted_draft_tokens == 0 and sampled.rejected_draft_tokens == 0     # not used for sampled requests


@pytest.mark.gpu
def test_predicted_outputs_on_gpu_are_lossless():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    prompt = list(range(10, 40))
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cuda", max_num_seqs=4, max_model_len=256))
    base = eng.generate([prompt], SamplingParams(max_tokens=40, temperature=0.0))[0]
    edited = list(base.output_ids)
    edited[7] = (edited[7] + 1) % 4000
    s0 = eng.step_count
    out = eng.generate([prompt], SamplingParams(max_tokens=40, temperature=0.0, prediction_ids=edited))[0]
    assert out.output_ids == base.output_ids
    assert out.accepted_draft_tokens >= 20 and out.rejected_draft_tokens > 0 and eng.step_count - s0 < 20


# ---------------------------------------------------------------- recurrent models: write-on-accept
def _hybrid_run(device, model, prompts, max_tokens=20, params=None, **kw):
    cfg = preset(model)
    eng = LLMEngine(EngineArgs(model=cfg, device=device, max_num_seqs=4, max_model_len=256, mtp_gate=False, **kw))
    if params is None:
        params = SamplingParams(max_tokens=max_tokens)
    outs = eng.generate(prompts, params)
    eng.last_outputs = outs
    return [o.output_ids for o in outs], eng


def _wrong_predictions(base):
    """The plain-decode output with every fifth token changed: predictions that are partly
    accepted and partly rejected, so the verify rows advance the recurrent state past what is
    finally committed."""
    preds = []
    for ids in base:
        p = list(ids)
        for j in range(4, len(p), 5):
            p[j] = (p[j] + 7) % 250 + 1
        preds.append(p)
    return preds


def _check_recurrent_speculation(device, model, **kw):
    prompts = [[3, 4, 5, 6, 3, 4, 5, 6, 3, 4, 5], [9, 8, 7, 9, 8, 7, 9, 8]]
    base, _ = _hybrid_run(device, model, prompts)
    # (1) predicted outputs with forced rejections
    params = [SamplingParams(max_tokens=20, prediction_ids=p) for p in _wrong_predictions(base)]
    got, eng = _hybrid_run(device, model, prompts, params=params, **kw)
    assert got == base
    assert sum(o.rejected_draft_tokens for o in eng.last_outputs) > 0       # rows past the accepted prefix were run
    assert sum(o.accepted_draft_tokens for o in eng.last_outputs) > 0
    # (2) n-gram drafts, whatever they are
    got, eng = _hybrid_run(device, model, prompts, speculative="ngram", num_drafts=3)
    assert got == base


@pytest.mark.parametrize("model", ["tiny-hybrid-moe", "tiny-nemotron-h", "tiny-kimi-linear"])
def test_speculation_on_recurrent_models_is_lossless_on_cpu(model):
    _check_recurrent_speculation("cpu", model)


@pytest.mark.gpu
@pytest.mark.parametrize("model", ["tiny-hybrid-moe", "tiny-nemotron-h", "tiny-kimi-linear"])
def test_speculation_on_recurrent_models_is_lossless_on_gpu(model):
    """Token-exact on the GPU as long as verify rows run on the kernel plain decode uses (up to 32
    query rows per KV head on the split-KV attention kernel: 3 drafts here). Wider verify steps
    take the split-Q attention kernel, whose summation order differs in the last bits, so a
    random-weight model may flip near-ties there; the recurrent state itself is compared bit for
    bit in tests/test_kernels_ext_gpu.py::test_write_on_accept_equals_feeding_only_the_accepted_rows."""
    _check_recurrent_speculation("cuda", model, prediction_drafts=3)


def test_mtp_k3_on_a_hybrid_model_is_lossless_on_cpu():
    prompts = [[3, 4, 5, 6, 3, 4, 5, 6, 3, 4, 5], [9, 8, 7, 9, 8, 7, 9, 8]]
    cfg = preset("tiny-hybrid-moe", mtp_layers=1)
    base = [o.output_ids for o in LLMEngine(EngineArgs(model=cfg, device="cpu", max_num_seqs=4, max_model_len=256,
                                                       mtp_gate=False)).generate(prompts, SamplingParams(max_tokens=16))]
    eng = LLMEngine(EngineArgs(model=cfg, device="cpu", max_num_seqs=4, max_model_len=256, mtp_gate=False,
                               speculative="mtp", num_drafts=3))
    got = [o.output_ids for o in eng.generate(prompts, SamplingParams(max_tokens=16))]
    assert got == base
    assert eng.spec_stats.drafted > 0


def _dflash_run(device, model="tiny-dense", **kw):
    eng = LLMEngine(EngineArgs(model=preset(model), device=device, max_num_seqs=4, max_model_len=256, mtp_gate=False,
                               speculative="dflash", **kw))
    outs = eng.generate(PROMPTS, SamplingParams(max_tokens=24))
    return [o.output_ids for o in outs], eng


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
def test_block_drafter_is_lossless_and_drafts_a_whole_block_per_forward(device):
    """DFlash-style drafter: every proposal is one drafter forward for all drafts of all
    sequences; whatever it drafts (random weights here), greedy output equals plain decoding."""
    base, _ = _run(device)
    got, eng = _dflash_run(device, dflash_gamma=4)
    assert got == base
    d = eng.runner.dflash
    assert eng.spec_stats.drafted > 0 and d.proposals > 0
    # several drafts per sequence per drafter forward (a step drafts for up to 3 sequences x 4)
    assert eng.spec_stats.drafted / d.proposals > 4


def test_block_drafter_context_follows_the_committed_tokens():
    """The drafter's context K/V of a position is a function of the committed prefix only: after
    speculative steps with rejected drafts it equals what a plain prefill of the same tokens writes
    (slots rewritten by the target are rewritten by the drafter in the same forward)."""
    import torch

    def run(prompt, n):
        eng = LLMEngine(EngineArgs(model=preset("tiny-dense"), device="cpu", max_num_seqs=4, max_model_len=256,
                                   mtp_gate=False, speculative="dflash", dflash_gamma=3, enable_prefix_caching=False))
        eng.add_request(prompt, SamplingParams(max_tokens=n))
        blocks, out = None, None
        while eng.has_work():
            for o in eng.step():
                if o.finished:
                    out = o.output_ids
            live = list(eng.scheduler.running) + list(eng.scheduler.prefilling)
            if live:
                blocks = list(live[0].blocks)
        return eng, blocks, out

    prompt = PROMPTS[0]
    eng_a, blocks_a, out = run(prompt, 12)                    # prefill + speculative decode steps
    assert eng_a.spec_stats.drafted > eng_a.spec_stats.accepted   # some drafts were rejected on the way
    full = prompt + out[:-1]
    eng_b, blocks_b, _ = run(full, 2)                         # the same tokens as one prefill (+ one decode step)
    bs = eng_a.runner.block_size
    for li in range(len(eng_a.runner.dflash.kv.k)):
        for name in ("k", "v"):
            a = getattr(eng_a.runner.dflash.kv, name)[li]
            b = getattr(eng_b.runner.dflash.kv, name)[li]
            a, b = a.reshape(-1, *a.shape[2:]), b.reshape(-1, *b.shape[2:])
            for p in range(len(full)):
                ra = a[blocks_a[p // bs] * bs + p % bs].float()
                rb = b[blocks_b[p // bs] * bs + p % bs].float()
                assert torch.allclose(ra, rb, atol=2e-2, rtol=2e-2), (li, name, p)
