"""The multi-stream residual highway: hyper-connection pre / post, engram and PLE gates, the dilated
convolution with carried state, n-gram hashing, and a dense model served over a four-stream highway."""
import torch

from metrale_inference_alpha_b200.engine.batch import ForwardBatch
from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.ops import highway as hw
from metrale_inference_alpha_b200.sampling.params import SamplingParams


def test_combination_matrix_is_doubly_stochastic_and_post_mixes_streams():
    g = torch.Generator().manual_seed(0)
    T, hc, H = 5, 4, 64
    streams = torch.randn(T, hc, H, generator=g)
    fn = (torch.randn((2 + hc) * hc, hc * H, generator=g) * 0.05).to(torch.bfloat16)
    scale, base = torch.tensor([1.0, 0.5, 2.0]), torch.randn((2 + hc) * hc, generator=g) * 0.1
    y, post, comb = hw.hc_pre(streams, fn, scale, base, iters=20)
    assert y.shape == (T, H) and post.shape == (T, hc) and comb.shape == (T, hc, hc)
    assert torch.allclose(comb.sum(1), torch.ones(T, hc), atol=1e-3) and torch.allclose(comb.sum(2), torch.ones(T, hc), atol=1e-2)
    assert (post > 0).all() and (post < 2).all()
    out = torch.randn(T, H, generator=g).to(torch.bfloat16)
    s2 = hw.hc_post(out, streams.clone(), post, comb)
    want = post[0, 1] * out[0].float() + sum(comb[0, i, 1] * streams[0, i] for i in range(hc))
    assert torch.allclose(s2[0, 1], want, atol=1e-5)
    # identity mixing leaves the streams alone apart from the block output
    eye = torch.eye(hc).expand(T, hc, hc).contiguous()
    s3 = hw.hc_post(out, streams.clone(), torch.zeros(T, hc), eye)
    assert torch.allclose(s3, streams)
    assert torch.equal(hw.hc_expand(out, hc)[:, 2], out.float()) and hw.hc_head_mean(hw.hc_expand(out, hc)).equal(out)


def test_engram_and_ple_gates_follow_their_formulas():
    g = torch.Generator().manual_seed(1)
    T, hc, H = 3, 2, 32
    streams = torch.randn(T, hc, H, generator=g)
    kv = torch.randn(T, (hc + 1) * H, generator=g).to(torch.bfloat16)
    qk = torch.rand(hc, H, generator=g)
    before = streams.clone()
    hw.engram_gate_add(streams, kv, qk)
    delta = streams - before
    val = kv[:, hc * H:].float()
    ratio = delta[1, 0] / val[1]
    assert torch.allclose(ratio, ratio[0].expand_as(ratio), atol=1e-4) and 0 < ratio[0] < 1      # one gate per (token, stream)
    key, value = torch.randn(T, hc * H, generator=g).to(torch.bfloat16), torch.randn(T, H, generator=g).to(torch.bfloat16)
    z = torch.zeros(hc, H)
    gated, normed = hw.ple_gate(before, key, value, z, z, z)
    g0 = gated.view(T, hc, H)[0, 1] / value[0].float()
    assert torch.allclose(g0, g0[0].expand_as(g0), atol=1e-4)
    assert torch.allclose(normed.view(T, hc, H).pow(2).mean(-1), torch.ones(T, hc), atol=1e-3)


def test_dilated_conv_state_carries_across_calls():
    g = torch.Generator().manual_seed(2)
    C, taps, dil, n = 6, 3, 2, 11
    x, base = torch.randn(n, C, generator=g), torch.randn(n, C, generator=g)
    w = torch.randn(C, taps, generator=g)
    def run(splits):
        state = torch.zeros(3, C, (taps - 1) * dil)
        outs, pos = [], 0
        for m in splits:
            b = ForwardBatch.build([dict(tokens=[1] * m, start_pos=pos, blocks=[1, 2], state_slot=1)], 16)
            outs.append(hw.dilated_conv(x[pos:pos + m], base[pos:pos + m], w, state, b, dil))
            pos += m
        return torch.cat(outs)
    whole = run([n])
    # by hand: row 5, channel 0
    acc = sum(w[0, j] * x[5 - (taps - 1 - j) * dil, 0] for j in range(taps))
    assert torch.allclose(whole[5, 0], base[5, 0] + torch.nn.functional.silu(acc), atol=1e-5)
    assert torch.allclose(run([4, 1, 1, 5]), whole, atol=1e-5) and torch.allclose(run([1] * n), whole, atol=1e-5)


def test_ngram_hash_ids_are_stable_and_depend_on_the_window():
    ids = hw.ngram_hash_ids([5, 6, 7, 5, 6, 7], n=3, table_rows=1000, cols=4)
    assert ids[2] == ids[5] and ids[1] != ids[2] and all(0 <= r < 1000 for row in ids for r in row)
    assert len({tuple(r) for r in ids}) >= 4 and len(set(ids[2])) > 1


def test_dense_model_on_a_four_stream_highway():
    prompts = [list(range(5, 60)), list(range(40, 52))]
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    whole = LLMEngine(EngineArgs(model="tiny-dense-hc", num_kv_blocks=64, max_num_seqs=4))
    want = [o.output_ids for o in whole.generate(prompts, sp)]
    chunked = LLMEngine(EngineArgs(model="tiny-dense-hc", num_kv_blocks=64, max_num_seqs=4, max_prefill_tokens=16))
    assert [o.output_ids for o in chunked.generate(prompts, sp)] == want
    assert all(L.hc_attn is not None and L.hc_ffn is not None for L in whole.weights.layers)
    assert whole.weights.layers[0].hc_attn[0].shape == (24, 4 * whole.cfg.hidden_size)
