"""Model families reached through config mapping and checkpoint-name dialects: Qwen2 (q/k/v bias),
Qwen3-MoE, Qwen2-MoE (shared expert + gate), Mixtral (block_sparse_moe / w1 w3 w2), Phi-3 (fused
qkv_proj / gate_up_proj), and text stacks wrapped under ``model.language_model.``. Each is checked
against a straight-line fp32 restatement of the HF forward pass written here from the tensors of
the checkpoint, not from the engine's decoder."""
import json
import math

import pytest
import torch
from safetensors.torch import save_file

from metrale_inference_alpha_b200.cache import KvCacheConfig, PagedKvCache
from metrale_inference_alpha_b200.config.model_config import from_hf_config
from metrale_inference_alpha_b200.engine.batch import ForwardBatch
from metrale_inference_alpha_b200.models.decoder import Decoder, LayerCaches
from metrale_inference_alpha_b200.weights.checkpoint import open_checkpoint
from metrale_inference_alpha_b200.weights.loader import load_weights
from metrale_inference_alpha_b200.weights.source import SyntheticSource

BASE = dict(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            head_dim=32, intermediate_size=256, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512,
            tie_word_embeddings=False)

FAMILIES = {
    "qwen2": dict(BASE, model_type="qwen2"),
    "qwen3_moe": dict(BASE, model_type="qwen3_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                      norm_topk_prob=True, decoder_sparse_step=1),
    "qwen2_moe": dict(BASE, model_type="qwen2_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                      shared_expert_intermediate_size=128, norm_topk_prob=False, decoder_sparse_step=1),
    "mixtral": dict(BASE, model_type="mixtral", num_local_experts=4, num_experts_per_tok=2, intermediate_size=64),
    "phi3": dict(BASE, model_type="phi3"),
}


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, theta):
    # x [T, H, D], rotate-half convention
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = pos[:, None].float() * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :], torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
    x1, x2 = x[..., :D // 2], x[..., D // 2:]
    return x * cos + torch.cat([-x2, x1], -1) * sin


def _oracle_logits(hf, get, has, toks):
    """fp32 forward of the whole sequence, HF semantics; `get(name)` returns a canonical tensor."""
    f = lambda n: get(n).float()
    T = len(toks)
    H, KV, D, eps = hf["num_attention_heads"], hf["num_key_value_heads"], hf["head_dim"], hf["rms_norm_eps"]
    mt = hf["model_type"]
    x = f("model.embed_tokens.weight")[torch.tensor(toks)]
    pos = torch.arange(T)
    for i in range(hf["num_hidden_layers"]):
        p = f"model.layers.{i}"
        a = _rms(x, f(f"{p}.input_layernorm.weight"), eps)
        q, k, v = (a @ f(f"{p}.self_attn.{n}_proj.weight").T for n in "qkv")
        if has(f"{p}.self_attn.q_proj.bias"):
            q, k, v = (t + f(f"{p}.self_attn.{n}_proj.bias") for t, n in zip((q, k, v), "qkv"))
        q, k, v = q.view(T, H, D), k.view(T, KV, D), v.view(T, KV, D)
        if has(f"{p}.self_attn.q_norm.weight"):
            q, k = _rms(q, f(f"{p}.self_attn.q_norm.weight"), eps), _rms(k, f(f"{p}.self_attn.k_norm.weight"), eps)
        q, k = _rope(q, pos, hf["rope_theta"]), _rope(k, pos, hf["rope_theta"])
        k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H * D)
        x = x + o @ f(f"{p}.self_attn.o_proj.weight").T
        a = _rms(x, f(f"{p}.post_attention_layernorm.weight"), eps)

        def mlp(q_, inp):
            g, u = inp @ f(f"{q_}.gate_proj.weight").T, inp @ f(f"{q_}.up_proj.weight").T
            return (torch.nn.functional.silu(g) * u) @ f(f"{q_}.down_proj.weight").T
        if has(f"{p}.mlp.gate.weight"):
            probs = (a @ f(f"{p}.mlp.gate.weight").T).softmax(-1)
            kx = hf["num_experts_per_tok"]
            w, idx = probs.topk(kx, -1)
            if mt == "mixtral" or hf.get("norm_topk_prob"):
                w = w / w.sum(-1, keepdim=True)
            y = torch.zeros_like(a)
            for t in range(T):
                for j in range(kx):
                    y[t] += w[t, j] * mlp(f"{p}.mlp.experts.{int(idx[t, j])}", a[t:t + 1])[0]
            if has(f"{p}.mlp.shared_expert.up_proj.weight"):
                sh = mlp(f"{p}.mlp.shared_expert", a)
                y = y + torch.sigmoid(a @ f(f"{p}.mlp.shared_expert_gate.weight").T) * sh
            x = x + y
        else:
            x = x + mlp(f"{p}.mlp", a)
    x = _rms(x, f("model.norm.weight"), eps)
    return x[-1] @ f("lm_head.weight").T


def _engine_logits(cfg, weights, toks):
    dec = Decoder(cfg, weights)
    kv = PagedKvCache(KvCacheConfig(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), 16)
    nb = (len(toks) + 15) // 16
    b = ForwardBatch.build([dict(tokens=toks, start_pos=0, blocks=list(range(1, nb + 1)))], 16)
    lg, _ = dec.forward(b, LayerCaches(cfg, kv=kv))
    return lg[0].float()


def _dialect(name: str, hf: dict, t: dict) -> dict:
    """Canonical tensors -> the spelling a real checkpoint of the family uses."""
    out = {}
    if name == "mixtral":
        ren = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}
        for n, v in t.items():
            n = n.replace(".mlp.gate.", ".block_sparse_moe.gate.")
            if ".mlp.experts." in n:
                n = n.replace(".mlp.experts.", ".block_sparse_moe.experts.")
                for a, b in ren.items():
                    n = n.replace(a, b)
            out[n] = v
        return out
    if name == "phi3":
        for n, v in t.items():
            if any(f".{x}_proj." in n for x in ("q", "k", "v", "gate", "up")):
                continue
            out[n] = v
        for i in range(hf["num_hidden_layers"]):
            p = f"model.layers.{i}"
            out[f"{p}.self_attn.qkv_proj.weight"] = torch.cat([t[f"{p}.self_attn.{x}_proj.weight"] for x in "qkv"])
            out[f"{p}.mlp.gate_up_proj.weight"] = torch.cat([t[f"{p}.mlp.{x}_proj.weight"] for x in ("gate", "up")])
        return out
    return dict(t)


@pytest.mark.parametrize("name", list(FAMILIES))
def test_family_matches_fp32_oracle_through_its_checkpoint_dialect(name, tmp_path):
    hf = FAMILIES[name]
    cfg = from_hf_config(hf, name=name)
    syn = SyntheticSource(cfg, seed=11, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    if name in ("qwen2", "qwen2_moe"):
        assert cfg.attn_bias and "model.layers.0.self_attn.q_proj.bias" in canon
    tensors = {k: v.contiguous() for k, v in _dialect(name, hf, canon).items()}
    if name == "qwen3_moe":                      # a text stack wrapped by a multimodal checkpoint
        tensors = {(("model.language_model." + k[len("model."):]) if k.startswith("model.") else k): v
                   for k, v in tensors.items()}
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(hf))
    cfg2, src = open_checkpoint(tmp_path)
    assert cfg2.arch == "dense_gqa" and cfg2.ffn_types == cfg.ffn_types
    w = load_weights(cfg2, src)
    toks = torch.randint(1, 512, (21,), generator=torch.Generator().manual_seed(5)).tolist()
    got = _engine_logits(cfg2, w, toks)
    want = _oracle_logits(hf, lambda n: canon[n], lambda n: n in canon, toks)
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert int(got.argmax()) == int(want.argmax())


def test_bias_is_not_silently_dropped():
    hf = FAMILIES["qwen2"]
    cfg = from_hf_config(hf)
    syn = SyntheticSource(cfg, seed=3, std=0.05)
    t = {n: syn.get(n) for n in syn.names()}
    from metrale_inference_alpha_b200.weights.source import DictSource
    toks = list(range(5, 20))
    a = _engine_logits(cfg, load_weights(cfg, DictSource(dict(t))), toks)
    for k in list(t):
        if k.endswith("_proj.bias"):
            t[k] = t[k] * 0 + 1.0
    b = _engine_logits(cfg, load_weights(cfg, DictSource(t)), toks)
    assert (a - b).abs().max() > 1e-3


def test_config_mapping_of_the_new_families():
    c = from_hf_config(dict(FAMILIES["qwen3_moe"], decoder_sparse_step=2, mlp_only_layers=[1]))
    assert c.ffn_types == ["dense", "dense"] and c.qk_norm and not c.attn_bias
    c = from_hf_config(FAMILIES["qwen2_moe"])
    assert c.num_shared_experts == 2 and c.shared_expert_gate and not c.router_renormalize and c.attn_bias
    c = from_hf_config(FAMILIES["mixtral"])
    assert c.num_experts == 4 and c.experts_per_token == 2 and c.moe_intermediate_size == 64 and c.router_renormalize
    with pytest.raises(ValueError):
        from_hf_config(dict(FAMILIES["phi3"], rope_scaling={"type": "longrope"}))
    c = from_hf_config(dict(FAMILIES["phi3"], partial_rotary_factor=0.5))
    assert c.rotary_dim == 16


GPU_BASE = dict(BASE, hidden_size=256, head_dim=64, intermediate_size=512, vocab_size=1024)


@pytest.mark.gpu
@pytest.mark.parametrize("name,extra", [
    ("qwen2", {}),
    ("qwen2_moe", dict(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                       shared_expert_intermediate_size=256, norm_topk_prob=False, decoder_sparse_step=1)),
    ("mixtral", dict(num_local_experts=4, num_experts_per_tok=2, intermediate_size=128)),
])
def test_family_on_gpu_matches_fp32_oracle(name, extra):
    """The same oracle against the CUDA decoder (bf16 weights through the tcgen05 GEMMs, the
    grouped expert GEMMs and the paged attention kernel)."""
    hf = dict(GPU_BASE, model_type=name, **extra)
    cfg = from_hf_config(hf, name=name)
    syn = SyntheticSource(cfg, seed=11, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    w = load_weights(cfg, syn, device="cuda:0")
    toks = torch.randint(1, 1024, (37,), generator=torch.Generator().manual_seed(5)).tolist()
    dec = Decoder(cfg, w)
    kv = PagedKvCache(KvCacheConfig(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), 16, device="cuda:0")
    nb = (len(toks) + 15) // 16
    b = ForwardBatch.build([dict(tokens=toks, start_pos=0, blocks=list(range(1, nb + 1)))], 16, device="cuda:0")
    lg, _ = dec.forward(b, LayerCaches(cfg, kv=kv))
    got = lg[0].float().cpu()
    want = _oracle_logits(hf, lambda n: canon[n], lambda n: n in canon, toks)
    err = (got - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item() + 1e-2, err


def test_checkpoint_preflight_reports_everything_at_once(tmp_path):
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.weights.preflight import preflight
    hf = FAMILIES["mixtral"]
    cfg = from_hf_config(hf, name="mixtral")
    syn = SyntheticSource(cfg, seed=1, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    tensors = {k: v.contiguous() for k, v in _dialect("mixtral", hf, canon).items()}
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(hf))
    cfg2, src = open_checkpoint(tmp_path)
    rep = preflight(cfg2, src)
    assert rep.ok and rep.checked > 40 and "present" in rep.summary()
    # break it: drop one expert projection and a norm, give another tensor the wrong shape
    bad = dict(tensors)
    del bad["model.layers.1.block_sparse_moe.experts.2.w3.weight"]
    del bad["model.layers.0.post_attention_layernorm.weight"]
    bad["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(7, 9, dtype=torch.bfloat16)
    d2 = tmp_path / "broken"
    d2.mkdir()
    save_file(bad, str(d2 / "model.safetensors"))
    (d2 / "config.json").write_text(json.dumps(hf))
    cfg3, src3 = open_checkpoint(d2)
    rep = preflight(cfg3, src3)
    assert not rep.ok and len(rep.missing) == 2 and len(rep.bad_shape) == 1
    text = rep.summary()
    assert "experts.2.up_proj" in text and "post_attention_layernorm" in text and "found (7, 9)" in text
    with pytest.raises(ValueError, match="preflight failed: 2 missing"):
        LLMEngine(EngineArgs(model=str(d2), device="cpu", max_num_seqs=2, max_model_len=64))
    from metrale_inference_alpha_b200.server.cli import main
    assert main(["preflight", str(tmp_path)]) == 0 and main(["preflight", str(d2)]) == 1


def test_arch_preflight_and_mxfp4_unpack():
    from metrale_inference_alpha_b200.ops import _native, reference as ref
    _native.check_arch((10, 0))
    with pytest.raises(RuntimeError, match="sm_100a"):
        _native.check_arch((9, 0))
    with pytest.raises(RuntimeError, match="sm_120"):
        _native.check_arch((12, 0))
    # e2m1 nibbles (low first) x 2^(e - 127) per 32 values
    codes = torch.arange(64, dtype=torch.uint8).remainder(16).view(1, 64)
    packed = ref.pack_fp4(codes)
    scales = torch.tensor([[127, 130]], dtype=torch.uint8)
    w = ref.dequantize_mxfp4(packed, scales)
    want = ref.e2m1_decode(codes).float() * torch.tensor([1.0] * 32 + [8.0] * 32)
    assert torch.equal(w, want) and w[0, 7] == 6.0 and w[0, 32 + 15] == -48.0
    assert torch.isnan(ref.e8m0_to_float(torch.tensor([255], dtype=torch.uint8)))[0]


GEMMA = dict(model_type="gemma3_text", vocab_size=512, hidden_size=128, num_hidden_layers=3, num_attention_heads=4,
             num_key_value_heads=2, head_dim=32, intermediate_size=256, rms_norm_eps=1e-6, rope_theta=1e6,
             rope_local_base_freq=1e4, sliding_window=8, sliding_window_pattern=3, query_pre_attn_scalar=64,
             max_position_embeddings=512, rope_scaling={"rope_type": "linear", "factor": 8.0},
             hidden_activation="gelu_pytorch_tanh", final_logit_softcapping=None, attn_logit_softcapping=None)


def _oracle_gemma(hf, get, toks):
    """fp32 Gemma 3 text forward: (1 + w) RMSNorm, scaled embeddings, sandwich norms, GeGLU, windowed
    layers with their own RoPE base, linearly scaled RoPE on the global layers, tied lm_head."""
    f = lambda n: get(n).float()
    T = len(toks)
    H, KV, D, eps = hf["num_attention_heads"], hf["num_key_value_heads"], hf["head_dim"], hf["rms_norm_eps"]
    rms = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w)

    def rope(x, pos, theta, factor):
        inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D)) / factor
        ang = pos[:, None].float() * inv[None, :]
        cos, sin = torch.cat([ang.cos()] * 2, -1)[:, None, :], torch.cat([ang.sin()] * 2, -1)[:, None, :]
        return x * cos + torch.cat([-x[..., D // 2:], x[..., :D // 2]], -1) * sin
    x = f("model.embed_tokens.weight")[torch.tensor(toks)] * torch.tensor(hf["hidden_size"] ** 0.5, dtype=torch.bfloat16).float()
    pos = torch.arange(T)
    for i in range(hf["num_hidden_layers"]):
        p = f"model.layers.{i}"
        local = (i + 1) % hf["sliding_window_pattern"] != 0
        a = rms(x, f(f"{p}.input_layernorm.weight"))
        q, k, v = ((a @ f(f"{p}.self_attn.{n}_proj.weight").T) for n in "qkv")
        q, k, v = q.view(T, H, D), k.view(T, KV, D), v.view(T, KV, D)
        q, k = rms(q, f(f"{p}.self_attn.q_norm.weight")), rms(k, f(f"{p}.self_attn.k_norm.weight"))
        theta, factor = (hf["rope_local_base_freq"], 1.0) if local else (hf["rope_theta"], hf["rope_scaling"]["factor"])
        q, k = rope(q, pos, theta, factor), rope(k, pos, theta, factor)
        k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = torch.einsum("thd,shd->hts", q, k) * hf["query_pre_attn_scalar"] ** -0.5
        mask = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
        if local:
            mask |= (pos[:, None] - pos[None, :]) >= hf["sliding_window"]
        o = torch.einsum("hts,shd->thd", s.masked_fill(mask, float("-inf")).softmax(-1), v).reshape(T, H * D)
        x = x + rms(o @ f(f"{p}.self_attn.o_proj.weight").T, f(f"{p}.post_attention_layernorm.weight"))
        a = rms(x, f(f"{p}.pre_feedforward_layernorm.weight"))
        g, u = a @ f(f"{p}.mlp.gate_proj.weight").T, a @ f(f"{p}.mlp.up_proj.weight").T
        y = (torch.nn.functional.gelu(g, approximate="tanh") * u) @ f(f"{p}.mlp.down_proj.weight").T
        x = x + rms(y, f(f"{p}.post_feedforward_layernorm.weight"))
    return rms(x, f("model.norm.weight"))[-1] @ f("model.embed_tokens.weight").T


def test_gemma3_text_matches_fp32_oracle(tmp_path):
    cfg = from_hf_config(GEMMA, name="gemma")
    assert cfg.window_layers == [8, 8, 0] and cfg.post_norms and cfg.ffn_act == "geglu" and cfg.tie_embeddings
    assert abs(cfg.attn_scale - 0.125) < 1e-9 and abs(cfg.embed_scale - 128 ** 0.5) < 1e-9 and cfg.rope_local_theta == 1e4
    syn = SyntheticSource(cfg, seed=4, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    assert "model.layers.0.pre_feedforward_layernorm.weight" in canon and "lm_head.weight" not in canon
    save_file({k: v.contiguous() for k, v in canon.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "gemma3", "text_config": GEMMA}))   # multimodal wrapper
    cfg2, src = open_checkpoint(tmp_path)
    w = load_weights(cfg2, src)
    toks = torch.randint(1, 512, (29,), generator=torch.Generator().manual_seed(2)).tolist()     # longer than the window
    got = _engine_logits(cfg2, w, toks)
    want = _oracle_gemma(GEMMA, lambda n: canon[n], toks)
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert int(got.argmax()) == int(want.argmax())
    with pytest.raises(ValueError, match="soft-capping"):
        from_hf_config(dict(GEMMA, model_type="gemma2", attn_logit_softcapping=50.0))
    capped = from_hf_config(dict(GEMMA, final_logit_softcapping=30.0))
    lg = _engine_logits(capped, load_weights(capped, src), toks)
    assert lg.abs().max() <= 30.0 and (lg - 30.0 * torch.tanh(got / 30.0)).abs().max() < 0.05


@pytest.mark.gpu
def test_gemma3_text_on_gpu_matches_fp32_oracle():
    hf = dict(GEMMA, hidden_size=256, head_dim=64, intermediate_size=512, vocab_size=1024, query_pre_attn_scalar=64)
    cfg = from_hf_config(hf, name="gemma")
    syn = SyntheticSource(cfg, seed=4, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    w = load_weights(cfg, syn, device="cuda:0")
    toks = torch.randint(1, 1024, (37,), generator=torch.Generator().manual_seed(2)).tolist()
    dec = Decoder(cfg, w)
    kv = PagedKvCache(KvCacheConfig(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), 16, device="cuda:0")
    nb = (len(toks) + 15) // 16
    b = ForwardBatch.build([dict(tokens=toks, start_pos=0, blocks=list(range(1, nb + 1)))], 16, device="cuda:0")
    lg, _ = dec.forward(b, LayerCaches(cfg, kv=kv))
    got = lg[0].float().cpu()
    want = _oracle_gemma(hf, lambda n: canon[n], toks)
    err = (got - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item() + 1e-2, err


GLM4 = dict(BASE, model_type="glm4", partial_rotary_factor=0.5, attention_bias=True)


def _oracle_glm4(hf, get, toks):
    """fp32 GLM-4 forward: q/k/v bias, interleaved rotary on the first half of each head, sandwich
    norms (no +1), SwiGLU from a fused gate_up projection."""
    f = lambda n: get(n).float()
    T = len(toks)
    H, KV, D, eps = hf["num_attention_heads"], hf["num_key_value_heads"], hf["head_dim"], hf["rms_norm_eps"]
    r = int(D * hf["partial_rotary_factor"])
    pos = torch.arange(T)
    inv = 1.0 / (hf["rope_theta"] ** (torch.arange(0, r, 2, dtype=torch.float32) / r))
    ang = pos[:, None].float() * inv[None, :]
    cos, sin = ang.cos().repeat_interleave(2, -1)[:, None, :], ang.sin().repeat_interleave(2, -1)[:, None, :]

    def rope(x):
        xr, xp = x[..., :r], x[..., r:]
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        rot = torch.stack([-x2, x1], -1).flatten(-2)
        return torch.cat([xr * cos + rot * sin, xp], -1)
    x = f("model.embed_tokens.weight")[torch.tensor(toks)]
    for i in range(hf["num_hidden_layers"]):
        p = f"model.layers.{i}"
        a = _rms(x, f(f"{p}.input_layernorm.weight"), eps)
        q, k, v = ((a @ f(f"{p}.self_attn.{n}_proj.weight").T + f(f"{p}.self_attn.{n}_proj.bias")) for n in "qkv")
        q, k, v = rope(q.view(T, H, D)), rope(k.view(T, KV, D)), v.view(T, KV, D)
        k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H * D)
        x = x + _rms(o @ f(f"{p}.self_attn.o_proj.weight").T, f(f"{p}.post_self_attn_layernorm.weight"), eps)
        a = _rms(x, f(f"{p}.post_attention_layernorm.weight"), eps)
        g, u = a @ f(f"{p}.mlp.gate_proj.weight").T, a @ f(f"{p}.mlp.up_proj.weight").T
        y = (torch.nn.functional.silu(g) * u) @ f(f"{p}.mlp.down_proj.weight").T
        x = x + _rms(y, f(f"{p}.post_mlp_layernorm.weight"), eps)
    return _rms(x, f("model.norm.weight"), eps)[-1] @ f("lm_head.weight").T


def test_glm4_matches_fp32_oracle(tmp_path):
    cfg = from_hf_config(GLM4, name="glm4")
    assert cfg.rope_interleaved and cfg.rotary_dim == 16 and cfg.post_norms and cfg.attn_bias and cfg.ffn_act == "swiglu"
    syn = SyntheticSource(cfg, seed=6, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    tensors = {}
    for n, v in canon.items():                      # the checkpoint stores gate and up as one gate_up_proj
        if ".mlp.gate_proj." in n or ".mlp.up_proj." in n:
            continue
        tensors[n] = v.contiguous()
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}.mlp"
        tensors[f"{p}.gate_up_proj.weight"] = torch.cat([canon[f"{p}.gate_proj.weight"], canon[f"{p}.up_proj.weight"]])
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(GLM4))
    cfg2, src = open_checkpoint(tmp_path)
    w = load_weights(cfg2, src)
    toks = torch.randint(1, 512, (23,), generator=torch.Generator().manual_seed(8)).tolist()
    got = _engine_logits(cfg2, w, toks)
    want = _oracle_glm4(GLM4, lambda n: canon[n], toks)
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert int(got.argmax()) == int(want.argmax())


MINIMAX = dict(BASE, model_type="minimax_m2", num_local_experts=8, num_experts_per_tok=2, intermediate_size=64,
               scoring_func="sigmoid", use_routing_bias=True, use_qk_norm=True, qk_norm_type="per_layer", rotary_dim=16)


def _oracle_minimax(hf, get, toks):
    """fp32 MiniMax-M2 forward: q / k RMSNorm over all heads jointly, partial NeoX rotary, MoE in every
    layer with sigmoid scores, selection by score + bias, weights = selected scores renormalised."""
    f = lambda n: get(n).float()
    T = len(toks)
    H, KV, D, eps, r = hf["num_attention_heads"], hf["num_key_value_heads"], hf["head_dim"], hf["rms_norm_eps"], hf["rotary_dim"]
    pos = torch.arange(T)
    inv = 1.0 / (hf["rope_theta"] ** (torch.arange(0, r, 2, dtype=torch.float32) / r))
    ang = pos[:, None].float() * inv[None, :]
    cos, sin = torch.cat([ang.cos()] * 2, -1)[:, None, :], torch.cat([ang.sin()] * 2, -1)[:, None, :]

    def rope(x):
        xr, xp = x[..., :r], x[..., r:]
        rot = torch.cat([-xr[..., r // 2:], xr[..., :r // 2]], -1)
        return torch.cat([xr * cos + rot * sin, xp], -1)
    x = f("model.embed_tokens.weight")[torch.tensor(toks)]
    for i in range(hf["num_hidden_layers"]):
        p = f"model.layers.{i}"
        a = _rms(x, f(f"{p}.input_layernorm.weight"), eps)
        q, k, v = ((a @ f(f"{p}.self_attn.{n}_proj.weight").T) for n in "qkv")
        q, k = _rms(q, f(f"{p}.self_attn.q_norm.weight"), eps), _rms(k, f(f"{p}.self_attn.k_norm.weight"), eps)
        q, k, v = rope(q.view(T, H, D)), rope(k.view(T, KV, D)), v.view(T, KV, D)
        k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        x = x + torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H * D) @ f(f"{p}.self_attn.o_proj.weight").T
        a = _rms(x, f(f"{p}.post_attention_layernorm.weight"), eps)
        scores = torch.sigmoid(a @ f(f"{p}.mlp.gate.weight").T)
        _, idx = (scores + f(f"{p}.mlp.gate.e_score_correction_bias")).topk(hf["num_experts_per_tok"], -1)
        w = scores.gather(1, idx)
        w = w / w.sum(-1, keepdim=True)
        y = torch.zeros_like(a)
        for t in range(T):
            for j in range(idx.shape[1]):
                e = f"{p}.mlp.experts.{int(idx[t, j])}"
                g, u = a[t] @ f(f"{e}.gate_proj.weight").T, a[t] @ f(f"{e}.up_proj.weight").T
                y[t] += w[t, j] * ((torch.nn.functional.silu(g) * u) @ f(f"{e}.down_proj.weight").T)
        x = x + y
    return _rms(x, f("model.norm.weight"), eps)[-1] @ f("lm_head.weight").T


def test_minimax_m2_matches_fp32_oracle(tmp_path):
    cfg = from_hf_config(MINIMAX, name="minimax")
    assert cfg.qk_norm_full and cfg.router == "sigmoid" and cfg.rotary_dim == 16 and cfg.ffn_types == ["moe", "moe"]
    syn = SyntheticSource(cfg, seed=9, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    assert canon["model.layers.0.self_attn.q_norm.weight"].shape == (128,) and canon["model.layers.0.self_attn.k_norm.weight"].shape == (64,)
    tensors = {}
    for n, v in _dialect("mixtral", MINIMAX, canon).items():       # same expert spelling as Mixtral ...
        n = n.replace(".block_sparse_moe.gate.e_score_correction_bias", ".block_sparse_moe.e_score_correction_bias")
        tensors[n] = v.contiguous()                                # ... and the routing bias beside the gate
    assert "model.layers.0.block_sparse_moe.e_score_correction_bias" in tensors
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(MINIMAX))
    cfg2, src = open_checkpoint(tmp_path)
    w = load_weights(cfg2, src)
    toks = torch.randint(1, 512, (19,), generator=torch.Generator().manual_seed(4)).tolist()
    got = _engine_logits(cfg2, w, toks)
    want = _oracle_minimax(MINIMAX, lambda n: canon[n], toks)
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert int(got.argmax()) == int(want.argmax())


def test_kimi_k2_maps_onto_the_deepseek_architecture():
    c = from_hf_config(dict(model_type="kimi_k2", vocab_size=1024, hidden_size=256, num_hidden_layers=3, num_attention_heads=4,
                            num_key_value_heads=4, intermediate_size=512, moe_intermediate_size=128, n_routed_experts=8,
                            num_experts_per_tok=2, n_shared_experts=1, first_k_dense_replace=1, kv_lora_rank=64, q_lora_rank=96,
                            qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, scoring_func="sigmoid", n_group=1,
                            topk_group=1, routed_scaling_factor=2.8, norm_topk_prob=True, rms_norm_eps=1e-6, rope_theta=5e4))
    assert c.arch == "deepseek_mla" and c.layer_types == ["mla"] * 3 and c.ffn_types == ["dense", "moe", "moe"]
    assert c.router == "sigmoid" and c.router_scaling == 2.8 and c.kv_lora_rank == 64 and c.head_dim == 48


@pytest.mark.gpu
def test_minimax_m2_on_gpu_matches_fp32_oracle():
    hf = dict(MINIMAX, hidden_size=512, head_dim=128, intermediate_size=128, vocab_size=1024, rotary_dim=64)   # the real head shape: 64 of 128 rotated
    cfg = from_hf_config(hf, name="minimax")
    syn = SyntheticSource(cfg, seed=9, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    w = load_weights(cfg, syn, device="cuda:0")
    toks = torch.randint(1, 1024, (33,), generator=torch.Generator().manual_seed(4)).tolist()
    dec = Decoder(cfg, w)
    kv = PagedKvCache(KvCacheConfig(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), 16, device="cuda:0")
    nb = (len(toks) + 15) // 16
    b = ForwardBatch.build([dict(tokens=toks, start_pos=0, blocks=list(range(1, nb + 1)))], 16, device="cuda:0")
    lg, _ = dec.forward(b, LayerCaches(cfg, kv=kv))
    got = lg[0].float().cpu()
    want = _oracle_minimax(hf, lambda n: canon[n], toks)
    err = (got - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item() + 1e-2, err


@pytest.mark.gpu
def test_glm4_on_gpu_matches_fp32_oracle():
    hf = dict(GLM4, hidden_size=512, head_dim=128, intermediate_size=512, vocab_size=1024)      # rotary 64 of 128, as in the real model
    cfg = from_hf_config(hf, name="glm4")
    syn = SyntheticSource(cfg, seed=6, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    w = load_weights(cfg, syn, device="cuda:0")
    toks = torch.randint(1, 1024, (35,), generator=torch.Generator().manual_seed(8)).tolist()
    dec = Decoder(cfg, w)
    kv = PagedKvCache(KvCacheConfig(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), 16, device="cuda:0")
    nb = (len(toks) + 15) // 16
    b = ForwardBatch.build([dict(tokens=toks, start_pos=0, blocks=list(range(1, nb + 1)))], 16, device="cuda:0")
    lg, _ = dec.forward(b, LayerCaches(cfg, kv=kv))
    got = lg[0].float().cpu()
    want = _oracle_glm4(hf, lambda n: canon[n], toks)
    err = (got - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item() + 1e-2, err


def test_olmo2_post_norm_only_matches_fp32_oracle():
    hf = dict(BASE, model_type="olmo2")
    cfg = from_hf_config(hf, name="olmo2")
    assert not cfg.pre_norms and cfg.post_norms and cfg.qk_norm_full
    syn = SyntheticSource(cfg, seed=12, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    assert "model.layers.0.input_layernorm.weight" not in canon and "model.layers.0.post_feedforward_layernorm.weight" in canon
    w = load_weights(cfg, syn)
    toks = torch.randint(1, 512, (17,), generator=torch.Generator().manual_seed(6)).tolist()
    got = _engine_logits(cfg, w, toks)
    f = lambda n: canon[n].float()
    T, H, KV, D, eps = len(toks), 4, 2, 32, hf["rms_norm_eps"]
    x = f("model.embed_tokens.weight")[torch.tensor(toks)]
    pos = torch.arange(T)
    for i in range(2):
        p = f"model.layers.{i}"
        q, k, v = ((x @ f(f"{p}.self_attn.{n}_proj.weight").T) for n in "qkv")
        q, k = _rms(q, f(f"{p}.self_attn.q_norm.weight"), eps), _rms(k, f(f"{p}.self_attn.k_norm.weight"), eps)
        q, k, v = _rope(q.view(T, H, D), pos, hf["rope_theta"]), _rope(k.view(T, KV, D), pos, hf["rope_theta"]), v.view(T, KV, D)
        k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H * D) @ f(f"{p}.self_attn.o_proj.weight").T
        x = x + _rms(o, f(f"{p}.post_attention_layernorm.weight"), eps)
        g, u = x @ f(f"{p}.mlp.gate_proj.weight").T, x @ f(f"{p}.mlp.up_proj.weight").T
        y = (torch.nn.functional.silu(g) * u) @ f(f"{p}.mlp.down_proj.weight").T
        x = x + _rms(y, f(f"{p}.post_feedforward_layernorm.weight"), eps)
    want = _rms(x, f("model.norm.weight"), eps)[-1] @ f("lm_head.weight").T
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert int(got.argmax()) == int(want.argmax())


def test_granite_multipliers_match_fp32_oracle():
    hf = dict(BASE, model_type="granite", embedding_multiplier=12.0, attention_multiplier=0.0625, residual_multiplier=0.22,
              logits_scaling=8.0)
    cfg = from_hf_config(hf, name="granite")
    assert cfg.embed_scale == 12.0 and cfg.attn_scale == 0.0625 and cfg.residual_multiplier == 0.22 and cfg.logits_divisor == 8.0
    syn = SyntheticSource(cfg, seed=13, std=0.05)
    canon = {n: syn.get(n) for n in syn.names()}
    toks = torch.randint(1, 512, (18,), generator=torch.Generator().manual_seed(7)).tolist()
    got = _engine_logits(cfg, load_weights(cfg, syn), toks)
    f = lambda n: canon[n].float()
    T, H, KV, D, eps = len(toks), 4, 2, 32, hf["rms_norm_eps"]
    x = f("model.embed_tokens.weight")[torch.tensor(toks)] * 12.0
    pos = torch.arange(T)
    for i in range(2):
        p = f"model.layers.{i}"
        a = _rms(x, f(f"{p}.input_layernorm.weight"), eps)
        q, k, v = ((a @ f(f"{p}.self_attn.{n}_proj.weight").T) for n in "qkv")
        q, k, v = _rope(q.view(T, H, D), pos, hf["rope_theta"]), _rope(k.view(T, KV, D), pos, hf["rope_theta"]), v.view(T, KV, D)
        k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = torch.einsum("thd,shd->hts", q, k) * 0.0625
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H * D) @ f(f"{p}.self_attn.o_proj.weight").T
        x = x + 0.22 * o
        a = _rms(x, f(f"{p}.post_attention_layernorm.weight"), eps)
        g, u = a @ f(f"{p}.mlp.gate_proj.weight").T, a @ f(f"{p}.mlp.up_proj.weight").T
        x = x + 0.22 * ((torch.nn.functional.silu(g) * u) @ f(f"{p}.mlp.down_proj.weight").T)
    want = (_rms(x, f("model.norm.weight"), eps)[-1] @ f("lm_head.weight").T) / 8.0
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert int(got.argmax()) == int(want.argmax())
