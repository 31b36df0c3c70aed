"""GGUF container, block dequantisers and the GGUF -> engine path."""
import numpy as np
import pytest
import torch

from metrale_inference_alpha_b200.config.model_config import preset
from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.sampling.params import SamplingParams
from metrale_inference_alpha_b200.weights import gguf
from metrale_inference_alpha_b200.weights.source import SyntheticSource


def test_container_roundtrip_and_block_quantisers(tmp_path):
    g = torch.Generator().manual_seed(0)
    a, b, c = torch.randn(8, 64, generator=g), torch.randn(4, 96, generator=g), torch.randn(5, generator=g)
    gguf.write_gguf(tmp_path / "t.gguf", {"general.architecture": "qwen3", "qwen3.block_count": 2, "x.f": 1.5, "x.s": "hi"},
                    {"a": (a, gguf.Q8_0), "b": (b, gguf.Q4_0), "c": (c, gguf.F32), "d": (a, gguf.F16)})
    f = gguf.GgufFile(tmp_path / "t.gguf")
    assert f.meta["qwen3.block_count"] == 2 and f.meta["x.s"] == "hi" and abs(f.meta["x.f"] - 1.5) < 1e-6
    assert f.tensors["a"][0] == (8, 64) and f.tensors["b"][0] == (4, 96)
    assert torch.equal(f.dequant("c"), c)
    assert torch.allclose(f.dequant("d"), a, atol=2e-3)
    assert (f.dequant("a") - a).abs().max() <= a.abs().max() / 127 * 0.51 + 1e-3       # Q8_0: half a step
    assert (f.dequant("b") - b).abs().max() <= b.abs().max() / 8 * 1.05 + 1e-3          # Q4_0: one step at the clipped end


def _scalar_q4_k(block: bytes) -> np.ndarray:
    """Independent scalar restatement of the Q4_K layout."""
    d, dmin = np.frombuffer(block[0:2], np.float16)[0].astype(np.float32), np.frombuffer(block[2:4], np.float16)[0].astype(np.float32)
    sc, qs = block[4:16], block[16:144]

    def scale_min(j):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
    out, o, is_ = np.zeros(256, np.float32), 0, 0
    for g0 in range(0, 128, 32):
        s1, m1 = scale_min(is_)
        s2, m2 = scale_min(is_ + 1)
        for l in range(32):
            out[o + l] = d * s1 * (qs[g0 + l] & 0xF) - dmin * m1
        for l in range(32):
            out[o + 32 + l] = d * s2 * (qs[g0 + l] >> 4) - dmin * m2
        o += 64
        is_ += 2
    return out


def _scalar_q6_k(block: bytes) -> np.ndarray:
    ql, qh = block[0:128], block[128:192]
    sc = np.frombuffer(block[192:208], np.int8)
    d = np.frombuffer(block[208:210], np.float16)[0].astype(np.float32)
    out = np.zeros(256, np.float32)
    for half in range(2):
        L, H, S, Y = ql[half * 64:], qh[half * 32:], sc[half * 8:], half * 128
        for l in range(32):
            i = l // 16
            q1 = ((L[l] & 0xF) | (((H[l] >> 0) & 3) << 4)) - 32
            q2 = ((L[l + 32] & 0xF) | (((H[l] >> 2) & 3) << 4)) - 32
            q3 = ((L[l] >> 4) | (((H[l] >> 4) & 3) << 4)) - 32
            q4 = ((L[l + 32] >> 4) | (((H[l] >> 6) & 3) << 4)) - 32
            out[Y + l] = d * S[i] * q1
            out[Y + l + 32] = d * S[i + 2] * q2
            out[Y + l + 64] = d * S[i + 4] * q3
            out[Y + l + 96] = d * S[i + 6] * q4
    return out


def test_k_quant_dequantisers_match_scalar_restatements():
    rng = np.random.default_rng(1)
    for typ, size, fn in ((gguf.Q4_K, 144, _scalar_q4_k), (gguf.Q6_K, 210, _scalar_q6_k)):
        raw = rng.integers(0, 256, size=(3, size), dtype=np.uint8)
        for r in raw:                                   # keep the f16 scale fields finite and small
            if typ == gguf.Q4_K:
                r[0:4] = np.array([0.01, 0.02], np.float16).view(np.uint8)
            else:
                r[208:210] = np.array([0.015], np.float16).view(np.uint8)
        got = gguf.dequantize(raw.reshape(-1), typ, 3 * 256).numpy().reshape(3, 256)
        want = np.stack([fn(bytes(r)) for r in raw])
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6), typ


def test_engine_runs_from_a_gguf_export_of_the_tiny_model(tmp_path):
    cfg = preset("tiny-dense", weight_format="bf16", qk_norm=False)
    src = SyntheticSource(cfg, seed=0)
    meta = {"general.architecture": "qwen2", "general.name": "tiny", "qwen2.block_count": cfg.num_layers,
            "qwen2.embedding_length": cfg.hidden_size, "qwen2.attention.head_count": cfg.num_heads,
            "qwen2.attention.head_count_kv": cfg.num_kv_heads, "qwen2.feed_forward_length": cfg.intermediate_size,
            "qwen2.rope.freq_base": float(cfg.rope_theta), "qwen2.attention.layer_norm_rms_epsilon": float(cfg.rms_eps),
            "qwen2.context_length": cfg.max_position, "qwen2.attention.key_length": cfg.head_dim}
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    for i in range(cfg.num_layers):
        p, q = f"model.layers.{i}", f"blk.{i}"
        names.update({f"{p}.input_layernorm.weight": f"{q}.attn_norm.weight",
                      f"{p}.post_attention_layernorm.weight": f"{q}.ffn_norm.weight",
                      f"{p}.self_attn.o_proj.weight": f"{q}.attn_output.weight"})
        for x in "qkv":
            names[f"{p}.self_attn.{x}_proj.weight"] = f"{q}.attn_{x}.weight"
        for x in ("gate", "up", "down"):
            names[f"{p}.mlp.{x}_proj.weight"] = f"{q}.ffn_{x}.weight"
    tensors = {}
    for hf, gg in names.items():
        if src.has(hf):
            t = src.get(hf).float()
            tensors[gg] = (t, gguf.F32 if t.ndim == 1 else gguf.Q8_0)
    gguf.write_gguf(tmp_path / "tiny.gguf", meta, tensors)
    s = gguf.GgufSource(tmp_path / "tiny.gguf")
    assert s.cfg.num_layers == cfg.num_layers and s.cfg.hidden_size == cfg.hidden_size and s.cfg.vocab_size == cfg.vocab_size
    w = src.get("model.layers.0.self_attn.q_proj.weight").float()
    assert (s.get("model.layers.0.self_attn.q_proj.weight").float() - w).abs().max() < w.abs().max() * 0.02
    eng = LLMEngine(EngineArgs(model=str(tmp_path / "tiny.gguf"), device="cpu", max_model_len=128))
    ref = LLMEngine(EngineArgs(model=cfg, device="cpu", max_model_len=128, seed=0))
    prompt = [[5, 6, 7, 8, 9]]
    a = eng.generate(prompt, SamplingParams(max_tokens=4))[0].output_ids
    b = ref.generate(prompt, SamplingParams(max_tokens=4))[0].output_ids
    assert len(a) == 4 and a[0] == b[0]                 # Q8_0 weights: the first greedy token survives
    assert gguf.hf_name("blk.3.attn_k_norm.weight") == "model.layers.3.self_attn.k_norm.weight"
    assert gguf.hf_name("rope_freqs.weight") is None


@pytest.mark.gpu
def test_device_dequantisers_match_the_host_ones(tmp_path):
    """Q8_0 / Q4_0 / Q4_K / Q6_K blocks widened by the device kernels equal the host dequantisation
    rounded to bf16, through the file path a loader takes (`GgufFile.dequant_device`)."""
    import torch
    rng = np.random.default_rng(5)
    sizes = {gguf.Q8_0: (32, 34), gguf.Q4_0: (32, 18), gguf.Q4_K: (256, 144), gguf.Q6_K: (256, 210)}
    for typ, (vals, size) in sizes.items():
        nb = 517
        raw = rng.integers(0, 256, size=(nb, size), dtype=np.uint8)
        for r in raw:                                   # finite, small f16 scale fields
            if typ in (gguf.Q8_0, gguf.Q4_0):
                r[0:2] = np.array([0.02], np.float16).view(np.uint8)
            elif typ == gguf.Q4_K:
                r[0:4] = np.array([0.01, 0.02], np.float16).view(np.uint8)
            else:
                r[208:210] = np.array([0.015], np.float16).view(np.uint8)
        want = gguf.dequantize(raw.reshape(-1), typ, nb * vals).to(torch.bfloat16)
        from metrale_inference_alpha_b200.ops import _native, _ptr, _stream
        dev_raw = torch.from_numpy(raw.reshape(-1).copy()).cuda()
        out = torch.empty(nb * vals, dtype=torch.bfloat16, device="cuda")
        _native.check(_native.lib().mb_gguf_dequant(typ, _ptr(dev_raw), nb, _ptr(out), _stream()), "gguf_dequant")
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), want), typ
