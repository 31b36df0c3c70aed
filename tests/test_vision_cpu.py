"""Vision input path: preprocessing, the ViT tower against the HF implementation of the same
architecture (random weights), and the multimodal rotary index."""
import base64
import io

import pytest
import torch

from metrale_inference_alpha_b200.vision import ImagePreprocessor, VisionConfig, VisionEncoder, mrope_positions, smart_resize
from metrale_inference_alpha_b200.vision.mrope import gather_tables
from metrale_inference_alpha_b200.vision.preprocess import decode_image


def test_smart_resize_bounds_and_multiples():
    assert smart_resize(224, 224) == (224, 224)
    h, w = smart_resize(1000, 700)
    assert h % 28 == 0 and w % 28 == 0 and abs(h / w - 1000 / 700) < 0.05
    h, w = smart_resize(4000, 6000, max_pixels=1_000_000)
    assert h * w <= 1_000_000 and h % 28 == 0
    h, w = smart_resize(20, 30)
    assert h * w >= 56 * 56
    with pytest.raises(ValueError):
        smart_resize(10, 5000)
    try:
        from transformers.models.qwen2_vl.image_processing_qwen2_vl import smart_resize as hf
    except Exception:
        return
    for hw in ((224, 224), (1000, 700), (333, 517), (20, 30), (3000, 2000)):
        assert smart_resize(*hw) == hf(*hw)


def test_patch_rows_are_in_merge_group_order_and_images_decode_from_data_urls():
    from PIL import Image
    import numpy as np
    pre = ImagePreprocessor()
    arr = (np.arange(56 * 84 * 3) % 251).astype("uint8").reshape(56, 84, 3)
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    assert torch.equal(decode_image(url), torch.from_numpy(arr))
    with pytest.raises(ValueError):
        decode_image("https://example.com/cat.png")
    rows, grid = pre([url])
    assert grid.tolist() == [[1, 4, 6]] and rows.shape == (24, 3 * 2 * 14 * 14)
    assert pre.num_image_tokens(56, 84) == 6
    # row 1 is the patch to the right of row 0 inside the first merge group; row 2 the one below row 0
    x = pre.resize_normalize(torch.from_numpy(arr))
    r = rows.view(24, 3, 2, 14, 14)
    assert torch.equal(r[0, :, 0], x[:, 0:14, 0:14]) and torch.equal(r[1, :, 0], x[:, 0:14, 14:28])
    assert torch.equal(r[2, :, 0], x[:, 14:28, 0:14]) and torch.equal(r[4, :, 0], x[:, 0:14, 28:42])
    assert torch.equal(r[0, :, 0], r[0, :, 1])                  # a still image fills the temporal patch with itself


def test_vision_tower_matches_the_hf_implementation():
    try:
        from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
        from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel
    except Exception as e:                                       # pragma: no cover
        pytest.skip(f"transformers vision tower unavailable: {e}")
    hf_cfg = Qwen2VLVisionConfig(depth=2, embed_dim=64, hidden_size=96, num_heads=4, mlp_ratio=2, in_channels=3,
                                 patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = Qwen2VisionTransformerPretrainedModel(hf_cfg).eval().float()
    cfg = VisionConfig(depth=2, embed_dim=64, hidden_size=96, num_heads=4, mlp_ratio=2)
    enc = VisionEncoder(cfg, {k: v.detach() for k, v in hf.state_dict().items()})
    grid = torch.tensor([[1, 4, 6], [2, 2, 4]])
    patches = torch.randn(24 + 16, cfg.patch_dim)
    with torch.no_grad():
        out = hf(patches, grid_thw=grid)
    want = out.pooler_output if getattr(out, "pooler_output", None) is not None else out
    if not isinstance(want, torch.Tensor):
        want = out[0]
    got = enc(patches, grid)
    assert got.shape == (10, 96)
    if want.shape != got.shape:                                  # some versions return the un-merged states first
        want = out.last_hidden_state if out.last_hidden_state.shape == got.shape else want
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), (got - want).abs().max()


def test_random_tower_shapes_and_argument_checks():
    cfg = VisionConfig(depth=1, embed_dim=32, hidden_size=48, num_heads=2, mlp_ratio=2)
    enc = VisionEncoder(cfg, VisionEncoder.random_tensors(cfg))
    grid = torch.tensor([[1, 2, 2]])
    assert enc(torch.randn(4, cfg.patch_dim), grid).shape == (1, 48)
    with pytest.raises(ValueError):
        enc(torch.randn(5, cfg.patch_dim), grid)
    with pytest.raises(ValueError):
        enc(torch.randn(4, 7), grid)


def test_mrope_positions_and_table_gather():
    IMG = 99
    toks = [1, 2] + [IMG] * 6 + [3, 4]                          # one image of 1 x 4 x 6 patches = 2 x 3 merged
    pos, delta = mrope_positions(toks, IMG, [(1, 4, 6)])
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8].tolist() == [5, 5, 5] and delta == -3
    assert int(pos.max()) + 1 == len(toks) + delta
    with pytest.raises(ValueError):
        mrope_positions([1, IMG, 2], IMG, [(1, 4, 6)])
    # text only: identical axes, so the gathered rows equal the plain table rows
    cos, sin = torch.rand(32, 8), torch.rand(32, 8)
    p, d = mrope_positions([5, 6, 7], IMG, [])
    c, s = gather_tables(cos, sin, p, [2, 3, 3])
    assert d == 0 and torch.equal(c, cos[:3]) and torch.equal(s, sin[:3])
    c, _ = gather_tables(cos, sin, pos, [2, 3, 3])
    assert torch.equal(c[4, :2], cos[2, :2]) and torch.equal(c[4, 2:5], cos[2, 2:5]) and torch.equal(c[4, 5:], cos[4, 5:])


# ----------------------------------------------------------------------------- images through the engine
def _vl_engine(**kw):
    import dataclasses
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    cfg = dataclasses.replace(preset("tiny-dense"), image_token_id=4000, vision_start_token_id=4001,
                              vision=dict(depth=1, embed_dim=32, num_heads=2, mlp_ratio=2), name="tiny-vl")
    eng = LLMEngine(EngineArgs(model=cfg, num_kv_blocks=128, max_num_seqs=4, max_model_len=512, **kw))
    eng.attach_vision()
    return eng


def _image(seed, h=56, w=84):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 255, (h, w, 3), generator=g, dtype=torch.uint8)


def test_images_reach_the_model_and_chunked_prefill_agrees():
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    prompt = list(range(5, 19)) + [4001, 4000, 7, 8, 9]         # one placeholder token per image
    a = _vl_engine()
    out1 = a.generate([prompt], sp, images=[[_image(1)]])[0]
    assert out1.prompt_tokens == len(prompt) - 1 + 6            # the placeholder expanded to 2 x 3 merged patches
    # the same picture again: served from the prefix cache, same tokens
    again = a.generate([prompt], sp, images=[[_image(1)]])[0]
    assert again.output_ids == out1.output_ids and again.cached_tokens > 0
    # a different picture must not reuse those cached blocks
    other = a.generate([prompt], sp, images=[[_image(3)]])[0]
    assert other.cached_tokens == 0
    b = _vl_engine(max_prefill_tokens=5)
    assert b.generate([prompt], sp, images=[[_image(1)]])[0].output_ids == out1.output_ids
    # text-only requests on the same engine behave as before
    t1 = a.generate([[5, 6, 7, 8]], sp)[0].output_ids
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    plain = LLMEngine(EngineArgs(model=preset("tiny-dense"), num_kv_blocks=128, max_num_seqs=4, max_model_len=512))
    assert plain.generate([[5, 6, 7, 8]], sp)[0].output_ids == t1


def test_image_rows_use_the_tower_embeddings_and_three_axis_positions():
    eng = _vl_engine()
    from metrale_inference_alpha_b200.engine.multimodal import build_inputs, expand_placeholders
    enc, pre = eng.vision
    ids, mm = build_inputs([1, 4000, 2], [_image(4)], encoder=enc, preprocessor=pre, image_token_id=4000, merge=2, device="cpu")
    assert ids == [1] + [4000] * 6 + [2] and mm.embeds.shape == (6, eng.cfg.hidden_size)
    assert mm.row_of_token == {i + 1: i for i in range(6)} and mm.delta == int(mm.positions.max()) + 1 - len(ids)
    assert mm.positions[1, 1:7].tolist() == [1, 1, 1, 2, 2, 2]
    assert expand_placeholders([1, 4000, 4000, 2], 4000, [2]) == [1, 4000, 4000, 2]
    with pytest.raises(ValueError):
        expand_placeholders([1, 2], 4000, [6])
    with pytest.raises(ValueError):
        eng.add_request([1, 2, 3], images=[_image(5)])


def test_vl_config_is_parsed():
    from metrale_inference_alpha_b200.config.model_config import from_hf_config
    cfg = from_hf_config({"model_type": "qwen2_vl", "hidden_size": 256, "num_hidden_layers": 2, "vocab_size": 1024,
                          "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 512,
                          "image_token_id": 1001, "vision_start_token_id": 1000,
                          "rope_scaling": {"type": "mrope", "mrope_section": [8, 12, 12]},
                          "vision_config": {"depth": 2, "embed_dim": 64, "num_heads": 4, "mlp_ratio": 2, "spatial_merge_size": 2}}, "vl")
    assert cfg.image_token_id == 1001 and cfg.mrope_sections == [8, 12, 12] and cfg.vision["depth"] == 2
    assert cfg.rope_scaling is None and cfg.attn_bias


def test_chat_completion_with_an_inline_image():
    import dataclasses
    import io
    import numpy as np
    from fastapi.testclient import TestClient
    from PIL import Image
    from metrale_inference_alpha_b200.config.model_config import preset
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
    from metrale_inference_alpha_b200.server.tokenizer import load_tokenizer
    tok = load_tokenizer(None, 4096)
    pad = tok.encode("<|image_pad|>")[0]
    cfg = dataclasses.replace(preset("tiny-dense"), image_token_id=pad, vision=dict(depth=1, embed_dim=32, num_heads=2, mlp_ratio=2),
                              name="tiny-vl")
    eng = LLMEngine(EngineArgs(model=cfg, num_kv_blocks=128, max_num_seqs=4, max_model_len=512))
    eng.attach_vision()
    buf = io.BytesIO()
    Image.fromarray((np.arange(56 * 56 * 3) % 255).astype("uint8").reshape(56, 56, 3)).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    with TestClient(create_app(eng, tok, ServerConfig(model_name="tiny-vl"))) as c:
        body = {"model": "tiny-vl", "max_tokens": 4, "temperature": 0,
                "messages": [{"role": "user", "content": [{"type": "text", "text": "what is this? "},
                                                            {"type": "image_url", "image_url": {"url": url}}]}]}
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        text_only = c.post("/v1/chat/completions", json=dict(body, messages=[{"role": "user", "content": "what is this? "}])).json()
        # the image expands to 2 x 2 merged patches between its start / end markers
        assert r.json()["usage"]["prompt_tokens"] == text_only["usage"]["prompt_tokens"] + 2 + 4
        bad = dict(body, messages=[{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "https://example.com/x.png"}}]}])
        assert c.post("/v1/chat/completions", json=bad).status_code == 400
    plain = LLMEngine(EngineArgs(model="tiny-dense", num_kv_blocks=64, max_num_seqs=2, max_model_len=256))
    with TestClient(create_app(plain, tok, ServerConfig(model_name="tiny"))) as c:
        assert c.post("/v1/chat/completions", json=dict(body, model="tiny")).status_code == 400


def test_media_integrity_gate_and_its_failure_classes():
    from metrale_inference_alpha_b200.bench.media_integrity import judge, media_integrity
    ok = [{"tokens": [1, 2], "cached_tokens": 0}, {"tokens": [1, 2], "cached_tokens": 32}, {"tokens": [3, 4], "cached_tokens": 16},
          {"tokens": [1, 2], "cached_tokens": 32}]
    assert judge(ok, placeholder_index=20, block_size=16)["pass"]
    crossed = [dict(r) for r in ok]
    crossed[2]["cached_tokens"] = 32
    assert "more than the 16" in judge(crossed, 20, 16)["why"]
    cold = [dict(r) for r in ok]
    cold[1]["cached_tokens"] = 0
    assert "did not hit" in judge(cold, 20, 16)["why"]
    drift = [dict(r) for r in ok]
    drift[3]["tokens"] = [1, 9]
    assert "same image differ" in judge(drift, 20, 16)["why"]
    blind = [dict(r) for r in ok]
    blind[2]["tokens"] = [1, 2]
    assert "does not depend" in judge(blind, 20, 16)["why"] and judge(blind, 20, 16, expect_different=False)["pass"]
    assert not judge(ok[:3], 20, 16)["pass"]
    eng = _vl_engine()
    prompt = list(range(5, 25)) + [4001, 4000] + list(range(30, 50))
    rec = media_integrity(eng, prompt, _image(1), _image(2), max_tokens=6, expect_different=False)
    assert rec.value == 1.0, rec.config
    assert rec.config["cached"][1] > 0 and rec.config["cached"][2] <= 16
    eng.close()
