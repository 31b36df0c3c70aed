"""Kimi delta attention: the per-channel gated delta rule, its chunked (UT-transform) form, the layer
inside the engine (chunked prefill carries the state; mixed with MLA layers) and the config parser."""
import torch

from metrale_inference_alpha_b200.config.model_config import from_hf_config
from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.ops import reference as ref
from metrale_inference_alpha_b200.sampling.params import SamplingParams


def _inputs(T, H, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = ref.l2_norm(torch.randn(T, H, D, generator=g))
    k = ref.l2_norm(torch.randn(T, H, D, generator=g))
    v = torch.randn(T, H, D, generator=g)
    gate = ref.kda_gate(torch.randn(T, H, D, generator=g), torch.randn(H, generator=g) * 0.3,
                        torch.randn(H, D, generator=g) * 0.3, -5.0)
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    return q, k, v, gate, beta


def test_gate_is_a_bounded_log_decay():
    g = ref.kda_gate(torch.randn(5, 2, 8) * 10, torch.zeros(2), torch.zeros(2, 8), -5.0)
    assert g.max() <= 0 and g.min() >= -5.0


def test_chunked_form_equals_the_token_recurrence():
    T, H, D = 70, 2, 32
    q, k, v, gate, beta = _inputs(T, H, D)
    S0 = torch.randn(1, H, D, D) * 0.1
    S, outs = S0.clone(), []
    for t in range(T):
        o, S = ref.kda_recurrence_step(S, q[t:t + 1], k[t:t + 1], v[t:t + 1], gate[t:t + 1], beta[t:t + 1])
        outs.append(o[0])
    for chunk in (16, 32, 64):
        o2, S2 = ref.kda_chunk(S0[0], q, k, v, gate, beta, chunk=chunk)
        assert torch.allclose(torch.stack(outs), o2, atol=1e-5) and torch.allclose(S[0], S2, atol=1e-5)


def test_a_zero_gate_reduces_to_the_plain_delta_rule():
    T, H, D = 9, 1, 16
    q, k, v, _, beta = _inputs(T, H, D, seed=1)
    S = torch.zeros(1, H, D, D)
    h = torch.zeros(1, H, D, D)
    for t in range(T):
        o, S = ref.kda_recurrence_step(S, q[t:t + 1], k[t:t + 1], v[t:t + 1], torch.zeros(1, H, D), beta[t:t + 1])
        o2, h = ref.gdn_recurrence_step(h, q[t:t + 1], k[t:t + 1], v[t:t + 1], torch.ones(1, H), beta[t:t + 1])
        assert torch.allclose(o, o2, atol=1e-6)


def test_chunked_prefill_carries_the_state():
    prompts = [list(range(5, 75)), list(range(40, 59))]
    sp = SamplingParams(max_tokens=5, temperature=0.0)
    whole = LLMEngine(EngineArgs(model="tiny-kimi-linear", num_kv_blocks=64, max_num_seqs=4))
    want = [o.output_ids for o in whole.generate(prompts, sp)]
    chunked = LLMEngine(EngineArgs(model="tiny-kimi-linear", num_kv_blocks=64, max_num_seqs=4, max_prefill_tokens=24))
    assert [o.output_ids for o in chunked.generate(prompts, sp)] == want


def test_kimi_linear_config_mixes_kda_with_position_free_mla():
    cfg = from_hf_config({"model_type": "kimi_linear", "hidden_size": 256, "num_hidden_layers": 4, "vocab_size": 2048,
                          "num_attention_heads": 4, "kv_lora_rank": 64, "qk_nope_head_dim": 32, "qk_rope_head_dim": 16,
                          "v_head_dim": 32, "mla_use_nope": True, "num_experts": 4, "num_experts_per_token": 2,
                          "moe_intermediate_size": 128, "intermediate_size": 256, "first_k_dense_replace": 1,
                          "num_shared_experts": 1,
                          "linear_attn_config": {"kda_layers": [1, 2, 3], "full_attn_layers": [4], "num_heads": 2,
                                                 "head_dim": 64, "short_conv_kernel_size": 4}}, "kl")
    assert cfg.layer_types == ["kda", "kda", "kda", "mla"] and cfg.rope_identity and cfg.kda_head_dim == 64
    eng = LLMEngine(EngineArgs(model=cfg, num_kv_blocks=64, max_num_seqs=2))
    # position-free: the rotary tables rotate by nothing
    assert torch.all(eng.runner.decoder.cos == 1) and torch.all(eng.runner.decoder.sin == 0)
    out = eng.generate([list(range(3, 40))], SamplingParams(max_tokens=4, temperature=0.0))[0].output_ids
    again = LLMEngine(EngineArgs(model=cfg, num_kv_blocks=64, max_num_seqs=2, max_prefill_tokens=16))
    assert again.generate([list(range(3, 40))], SamplingParams(max_tokens=4, temperature=0.0))[0].output_ids == out
