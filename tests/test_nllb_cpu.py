"""NLLB / M2M-100 encoder-decoder: logits against the HF implementation of the same architecture (random
weights), incremental decoding against teacher forcing, and beam search."""
import pytest
import torch

from metrale_inference_alpha_b200.models.nllb import NllbConfig, NllbModel, sinusoidal_table


def _hf(seed=0):
    try:
        from transformers import M2M100Config, M2M100ForConditionalGeneration
    except Exception as e:                                       # pragma: no cover
        pytest.skip(f"transformers M2M100 unavailable: {e}")
    torch.manual_seed(seed)
    hc = M2M100Config(vocab_size=200, d_model=64, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                      decoder_attention_heads=4, encoder_ffn_dim=128, decoder_ffn_dim=128, max_position_embeddings=128,
                      scale_embedding=True, pad_token_id=1, bos_token_id=0, eos_token_id=2, decoder_start_token_id=2)
    m = M2M100ForConditionalGeneration(hc).eval()
    cfg = NllbConfig.from_hf(hc.to_dict())
    return m, NllbModel(cfg, {k: v.detach() for k, v in m.state_dict().items()})


def test_position_table_skips_the_padding_row():
    tab = sinusoidal_table(10, 8, 1)
    assert torch.count_nonzero(tab[1]) == 0 and torch.allclose(tab[0, 4:], torch.ones(4)) and tab.shape == (10, 8)


def test_logits_match_the_hf_model_with_padding_and_incremental_decoding():
    hf, mine = _hf()
    src = torch.tensor([[10, 11, 12, 13, 2], [10, 44, 2, 1, 1]])
    dec = torch.tensor([[2, 20, 31, 32, 33], [2, 20, 41, 42, 43]])
    with torch.no_grad():
        want = hf(input_ids=src, attention_mask=(src != 1).long(), decoder_input_ids=dec).logits
    enc = mine.encode(src)
    got = mine.decode_step(dec, enc, mine.new_cache(), 0)
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), (got - want).abs().max()
    # token by token over the cache = teacher forcing
    cache, outs = mine.new_cache(), []
    for t in range(dec.shape[1]):
        outs.append(mine.decode_step(dec[:, t:t + 1], enc, cache, t))
    assert torch.allclose(torch.cat(outs, 1), got, atol=1e-4)


@pytest.mark.parametrize("beams", [1, 3])
def test_translation_follows_hf_generate(beams):
    hf, mine = _hf(1)
    for src in ([10, 11, 12, 13, 2], [10, 90, 91, 92, 93, 94, 2]):
        with torch.no_grad():
            want = hf.generate(torch.tensor([src]), forced_bos_token_id=20, num_beams=beams, max_new_tokens=10,
                               length_penalty=1.0, early_stopping=False, do_sample=False)[0].tolist()
        got = mine.translate(src, 20, num_beams=beams, max_new_tokens=10)
        want_body = [t for t in want[2:] if t not in (1, 2)]
        if got != want_body:
            # both searches are heuristic about when to stop: ours must then be at least as good under the shared score
            def score(body):
                ids = torch.tensor([[2, 20] + body + [2]])
                lp = torch.log_softmax(mine.decode_step(ids[:, :-1], mine.encode(torch.tensor([src])), mine.new_cache(), 0), -1)
                tok = lp[0, torch.arange(ids.shape[1] - 1), ids[0, 1:]]
                return float(tok[1:].sum()) / ids.shape[1]
            assert score(got) >= score(want_body) - 1e-4
        assert len(got) <= 10 and 2 not in got


def test_budget_closes_every_beam():
    _, mine = _hf(2)
    out = mine.translate([10, 11, 2], 20, num_beams=2, max_new_tokens=3)
    assert len(out) <= 3


def test_translation_routes_and_checkpoint_loading(tmp_path):
    import json
    from fastapi.testclient import TestClient
    from safetensors.torch import save_file
    from metrale_inference_alpha_b200.server.translate import (Translator, create_translation_app, is_translation_checkpoint,
                                                                open_translation_model)
    hf, mine = _hf(3)
    d = tmp_path / "nllb"
    d.mkdir()
    cfgd = hf.config.to_dict()
    (d / "config.json").write_text(json.dumps(cfgd))
    sd = {k: v.detach().clone().contiguous() for k, v in hf.state_dict().items() if k not in ("lm_head.weight", "model.encoder.embed_tokens.weight", "model.decoder.embed_tokens.weight")}
    save_file(sd, str(d / "model.safetensors"))
    assert is_translation_checkpoint(d) and not is_translation_checkpoint(tmp_path)
    model, _ = open_translation_model(d)

    class Tok:                                                   # bytes 3..199 as ids; language codes as fixed ids
        unk_token_id = 3
        def encode(self, s): return [4 + (b % 150) for b in s.encode()]
        def decode(self, ids): return " ".join(str(i) for i in ids)
        def convert_tokens_to_ids(self, t): return {"eng_Latn": 10, "fra_Latn": 20}.get(t, 3)

    tr = Translator(model, Tok(), "eng_Latn", "fra_Latn", num_beams=2)
    direct = model.translate([10] + Tok().encode("hi there.") + [2], 20, num_beams=2, max_new_tokens=6)
    with TestClient(create_translation_app(tr, "nllb-tiny")) as c:
        assert c.get("/health").json()["task"] == "translation"
        r = c.post("/v1/completions", json={"prompt": "hi there.", "max_tokens": 6}).json()
        assert r["choices"][0]["text"] == Tok().decode(direct) and r["usage"]["completion_tokens"] == len(direct)
        r2 = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi there. and more!"}], "max_tokens": 4})
        assert r2.status_code == 200 and r2.json()["choices"][0]["message"]["role"] == "assistant"
        assert c.post("/v1/completions", json={"prompt": "x", "tgt_lang": "xxx_Latn"}).status_code == 400
        assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
